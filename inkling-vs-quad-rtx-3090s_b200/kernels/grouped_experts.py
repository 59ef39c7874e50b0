"""Grouped expert projections over checkpoint-layout NVFP4 weights, and the bank naming
shared with the decode path. `expert_gemm[grid](...)` and `expert_reduce[grid](...)` keep
the launch syntax and argument lists of the reference's Triton kernels
(kernels/grouped_experts.py:26-43, :152-163)."""
from __future__ import annotations

import torch

from . import _abi
from .expert_planner import _Launcher


def expert_bank_names(quantized: bool) -> list[str]:
    """One expert's weight banks in pointer-table order (reference:
    kernels/grouped_experts.py:9-22): gate/up first, then down, each followed by its
    NVFP4 scale banks when quantized. The length is the pointer-table stride."""
    suffixes = ("", "_scale", "_scale2") if quantized else ("",)
    return [projection + suffix for projection in ("gate_up_proj", "down_proj") for suffix in suffixes]


_SCRATCH: dict[tuple, torch.Tensor] = {}


def _scratch(rows: int, device) -> torch.Tensor:
    """Per-device buffer for the activations' row normalisers; grows to the largest
    request and is then reused, so a captured step never allocates."""
    key = (device.type, device.index)
    need = _abi.lib().ink_expert_gemm_scratch_bytes(rows)
    buf = _SCRATCH.get(key)
    if buf is None or buf.numel() < need:
        buf = torch.empty(max(need, 1 << 16), dtype=torch.uint8, device=device)
        _SCRATCH[key] = buf
    return buf


def _expert_gemm(X, Pointers, Experts, Rows, Counts, Y, CAPACITY, N, K, TOP_K, PROJECTION, QUANTIZED, STRIDE,
                 BM=None, BN=None, BK=None, groups=None, status=None):
    """One projection for every active expert's routed rows. Arguments as the reference's
    expert_gemm; BM/BN/BK (Triton tile sizes) are ignored, `groups` defaults to every
    entry of Experts (the reference passes the bound through its grid)."""
    assert X.dtype == Y.dtype == torch.bfloat16 and X.is_contiguous() and Y.is_contiguous()
    assert Experts.dtype == Counts.dtype == Rows.dtype == torch.int32 and Pointers.dtype == torch.int64
    assert STRIDE == len(expert_bank_names(bool(QUANTIZED))) and X.shape[1] == K
    _abi.require_cuda(X, Pointers, Experts, Rows, Counts, Y)
    groups = Experts.numel() if groups is None else groups
    scratch = _scratch(X.shape[0], X.device)
    _abi.check(_abi.lib().ink_expert_gemm(
        X.data_ptr(), X.shape[0], Pointers.data_ptr(), Experts.data_ptr(), Rows.data_ptr(), Counts.data_ptr(),
        Y.data_ptr(), CAPACITY, N, K, TOP_K, PROJECTION, int(bool(QUANTIZED)), groups, scratch.data_ptr(),
        scratch.numel(), _abi.ptr(status), _abi.stream()))


def _expert_reduce(Down, Indices, Weights, Pointers, Output, WIDTH, TOP_K, POINTER_STRIDE, MAX_EXPERT, BLOCK=None):
    """Add each token's routed expert outputs, scaled by the router weights, to Output;
    routes whose pointer row is zero are skipped. Arguments as the reference's expert_reduce."""
    assert Down.dtype == Weights.dtype == torch.bfloat16 and Output.dtype == torch.float32
    assert Indices.dtype == Pointers.dtype == torch.int64
    _abi.require_cuda(Down, Indices, Weights, Pointers, Output)
    tokens = Indices.shape[0]
    _abi.check(_abi.lib().ink_expert_reduce(
        Down.data_ptr(), Indices.data_ptr(), Weights.data_ptr(), Pointers.data_ptr(), Output.data_ptr(), tokens,
        WIDTH, TOP_K, POINTER_STRIDE, MAX_EXPERT, _abi.stream()))


class _GemmLauncher(_Launcher):
    """`expert_gemm[grid](...)`: the third grid dimension is the number of groups to visit,
    as in the reference's launch (my_inkling/offloaded_experts.py:262)."""

    def __getitem__(self, grid):
        groups = grid[2] if isinstance(grid, (tuple, list)) and len(grid) > 2 else None
        return lambda *args, **kwargs: self._fn(*args, groups=groups, **kwargs)


expert_gemm = _GemmLauncher(_expert_gemm)
expert_reduce = _Launcher(_expert_reduce)
