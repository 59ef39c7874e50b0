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


def _scratch(rows: int, device, k: int = 0) -> torch.Tensor:
    """Per-device buffer for the activations' row normalisers (and, for the block-scaled
    kernel, their digit rows: pass `k`); grows to the largest request and is then reused, so
    a captured step never allocates once it has been warmed up at its largest shape."""
    key = (device.type, device.index)
    need = _abi.lib().ink_expert_gemm_tc_scratch_bytes(rows, k) if k else _abi.lib().ink_expert_gemm_scratch_bytes(rows)
    buf = _SCRATCH.get(key)
    if buf is None or buf.numel() < need:
        buf = torch.empty(max(need, 1 << 16), dtype=torch.uint8, device=device)
        _SCRATCH[key] = buf
    return buf


def encode_bank_maps(layout, experts: int, hidden: int, intermediate: int, device) -> torch.Tensor:
    """The four TMA descriptors of one layer's evenly spaced NVFP4 banks as a 512-byte device
    tensor (ink_moe_stack_encode_banks). `layout` = ((address of expert 0, byte distance between
    experts) for gate_up_proj, gate_up_proj_scale, down_proj, down_proj_scale)."""
    import ctypes

    host = bytearray(512)
    out = (ctypes.c_char * 512).from_buffer(host)
    (gc, gcs), (gs, gss), (dc, dcs), (ds, dss) = layout
    _abi.check(_abi.lib().ink_moe_stack_encode_banks(out, gc, gcs, gs, gss, dc, dcs, ds, dss, experts, hidden, intermediate))
    maps = torch.frombuffer(host, dtype=torch.uint8).to(device)
    assert maps.data_ptr() % 128 == 0
    return maps


def block_scaled_supported(n: int, k: int, groups: int) -> bool:
    """Shapes the block-scaled tensor-core kernel takes (ink_expert_gemm_tc)."""
    return n % 128 == 0 and k % 256 == 0 and 256 <= k <= 4096 and groups <= 1024


def _expert_gemm(X, Pointers, Experts, Rows, Counts, Y, CAPACITY, N, K, TOP_K, PROJECTION, QUANTIZED, STRIDE,
                 BM=None, BN=None, BK=None, groups=None, status=None, bank_maps=None, start: int = 0):
    """One projection for every active expert's routed rows. Arguments as the reference's
    expert_gemm; BM/BN/BK (Triton tile sizes) are ignored, `groups` defaults to every
    entry of Experts (the reference passes the bound through its grid). With `bank_maps` (the
    layer's TMA descriptors, see encode_bank_maps; `start` = id of the first expert they cover)
    the projection runs on the block-scaled tensor-core kernel, which reads the packed banks as
    they are; without, on the kernel that expands them to FP16 first."""
    assert X.dtype == Y.dtype == torch.bfloat16 and X.is_contiguous() and Y.is_contiguous()
    assert Experts.dtype == Counts.dtype == Rows.dtype == torch.int32 and Pointers.dtype == torch.int64
    assert STRIDE == len(expert_bank_names(bool(QUANTIZED))) and X.shape[1] == K
    _abi.require_cuda(X, Pointers, Experts, Rows, Counts, Y)
    groups = Experts.numel() if groups is None else groups
    if bank_maps is not None and QUANTIZED and block_scaled_supported(N, K, groups):
        scratch = _scratch(X.shape[0], X.device, K)
        _abi.check(_abi.lib().ink_expert_gemm_tc(
            X.data_ptr(), X.shape[0], bank_maps.data_ptr(), Pointers.data_ptr(), Experts.data_ptr(), Rows.data_ptr(),
            Counts.data_ptr(), Y.data_ptr(), CAPACITY, N, K, TOP_K, PROJECTION, groups, start, scratch.data_ptr(),
            scratch.numel(), _abi.ptr(status), _abi.stream()))
        return
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
