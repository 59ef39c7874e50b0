"""Routed-expert projections for a few tokens: one matrix-vector product per route.

Same call as the reference's kernels/routed_decode.py:25-80, served by the sm_100a
library (gate_up and down_reduce of kernels/routed_decode.cu:137-219).
"""
from __future__ import annotations

import torch

from . import _abi


def routed_decode(x, indices, weights, pointers, activated, output, max_expert: int, quantized: bool,
                  rows: int | None = None, status: torch.Tensor | None = None) -> None:
    """output[token] = sum over its routes of weight * down(silu(gate) * up).

    Routes whose pointer-table row is zero (experts of other ranks) are skipped.
    `activated` is scratch for the intermediate; `output` is overwritten. `rows` (the
    reference's tiling knob) is accepted and ignored: tiling is fixed per width here.
    `status` (optional int32[1]) gets bit 0 set if a route names an expert outside
    [0, max_expert].
    """
    tokens, hidden = x.shape
    top_k = indices.shape[1]
    intermediate = activated.shape[1]
    assert x.dtype == activated.dtype == weights.dtype == torch.bfloat16
    assert indices.dtype == pointers.dtype == torch.int64
    assert output.dtype == torch.float32 and output.shape == x.shape
    assert all(t.is_contiguous() and t.data_ptr() % 16 == 0 for t in (x, indices, weights, activated, output))
    assert activated.shape[0] >= tokens * top_k
    _abi.require_cuda(x, indices, weights, pointers, activated, output)
    _abi.check(_abi.lib().ink_routed_decode(
        x.data_ptr(), indices.data_ptr(), weights.data_ptr(), pointers.data_ptr(), activated.data_ptr(),
        output.data_ptr(), tokens, top_k, hidden, intermediate, max_expert, int(bool(quantized)),
        _abi.ptr(status), _abi.stream()))


def moe_decode(x, indices, weights, pointers, activated, shared_gate, shared_up, shared_down, gammas,
               shared_activated, output, max_expert: int, status: torch.Tensor | None = None,
               half: str = "both") -> None:
    """Routed NVFP4 experts plus the shared BF16 experts of one layer, FP32 partial sum
    into `output` (fully overwritten). Shapes as in include/inkling_b200.h. `half` picks
    one of the two launches ("gate_up", "down") or "both"."""
    tokens, hidden = x.shape
    top_k = indices.shape[1]
    intermediate = activated.shape[1]
    n_shared = shared_gate.shape[0]
    assert x.dtype == activated.dtype == weights.dtype == gammas.dtype == torch.bfloat16
    assert shared_gate.dtype == shared_up.dtype == shared_down.dtype == shared_activated.dtype == torch.bfloat16
    assert shared_gate.shape == shared_up.shape == (n_shared, intermediate, hidden)
    assert shared_down.shape == (n_shared, hidden, intermediate)
    assert gammas.shape == (tokens, n_shared) and shared_activated.shape[0] >= tokens * n_shared
    assert indices.dtype == pointers.dtype == torch.int64
    assert output.dtype == torch.float32 and output.shape == x.shape
    tensors = (x, indices, weights, activated, output, shared_gate, shared_up, shared_down, gammas, shared_activated)
    assert all(t.is_contiguous() for t in tensors)
    _abi.require_cuda(*tensors, pointers)
    fn = {"both": "ink_moe_decode", "gate_up": "ink_moe_gate_up", "down": "ink_moe_down"}[half]
    _abi.check(getattr(_abi.lib(), fn)(
        x.data_ptr(), indices.data_ptr(), weights.data_ptr(), pointers.data_ptr(), activated.data_ptr(),
        shared_gate.data_ptr(), shared_up.data_ptr(), shared_down.data_ptr(), gammas.data_ptr(),
        shared_activated.data_ptr(), output.data_ptr(), tokens, top_k, n_shared, hidden, intermediate,
        max_expert, _abi.ptr(status), _abi.stream()))


def add_rmsnorm(partial, residual, weight, eps: float, normed) -> None:
    """residual += bf16(partial) (BF16 add), normed = rms_norm(residual) * weight with the
    reference's rounding (kernels/decode.py:36-43). In place on `residual`."""
    tokens, hidden = partial.shape
    assert partial.dtype == torch.float32 and residual.dtype == weight.dtype == normed.dtype == torch.bfloat16
    assert residual.shape == normed.shape == partial.shape and weight.shape == (hidden,)
    assert all(t.is_contiguous() for t in (partial, residual, weight, normed))
    _abi.require_cuda(partial, residual, weight, normed)
    _abi.check(_abi.lib().ink_add_rmsnorm(partial.data_ptr(), residual.data_ptr(), weight.data_ptr(), float(eps),
                                          normed.data_ptr(), tokens, hidden, _abi.stream()))


def short_conv(x, weight, history, residual=None):
    """One decode token through the short convolution, as the reference's
    kernels/decode.py:115-146 `short_conv`: x [bs, 1, d] BF16 (or FP32: the block's all-reduced
    output, rounded to BF16 first), weight FP32 [d, 1, K], history FP32 [bs, d, K] shifted in
    place, residual [bs, 1, d] BF16 or None. Returns BF16 [bs, 1, d]."""
    bs, _, d = x.shape
    k = weight.shape[-1]
    assert x.stride(-1) == 1 and x.is_contiguous() and history.is_contiguous() and weight.is_contiguous()
    assert x.dtype in (torch.bfloat16, torch.float32) and weight.dtype == history.dtype == torch.float32
    assert history.shape == (bs, d, k) and weight.shape == (d, 1, k)
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == x.shape and residual.is_contiguous()
    y = torch.empty((bs, 1, d), dtype=torch.bfloat16, device=x.device)
    _abi.require_cuda(x, weight, history, residual, y)
    _abi.check(_abi.lib().ink_short_conv(x.data_ptr(), int(x.dtype == torch.float32), weight.data_ptr(),
                                         history.data_ptr(), _abi.ptr(residual), y.data_ptr(), bs, d, k,
                                         _abi.stream()))
    return y
