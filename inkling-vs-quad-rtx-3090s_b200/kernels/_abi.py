"""ctypes binding of the C ABI in include/inkling_b200.h.

The library is built ahead of time by csrc/build.py and lives next to this package.
There is no fallback: if it is missing, loading fails with the build command to run.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_size_t, c_void_p
from pathlib import Path

import torch

LIBRARY = Path(__file__).resolve().parents[1] / "libinkling_b200.so"
ABI_VERSION = 1
_lib = None

P, I, F, Z = c_void_p, c_int, c_float, c_size_t
_SIGNATURES = {
    "ink_last_error": (c_char_p, []),
    "ink_abi_version": (I, []),
    "ink_router_workspace_bytes": (Z, [I, I]),
    "ink_router_forward": (I, [P, P, P, P, F, I, I, I, I, I, P, P, P, P, P, Z, P]),
    "ink_router_forward_static": (I, [P, P, P, P, F, I, I, I, I, I, P, P, P, P, P]),
    "ink_router_plan_forward": (I, [P, P, P, P, F, I, I, I, I, I, P, P, P, P, P, Z,
                                    P, P, P, P, P, I, I, I, I, P]),
    "ink_expert_plan": (I, [P, P, P, P, P, P, I, I, I, I, I, P]),
    "ink_routed_decode": (I, [P, P, P, P, P, P, I, I, I, I, I, I, P, P]),
    "ink_moe_decode": (I, [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, P, P]),
    "ink_moe_gate_up": (I, [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, P, P]),
    "ink_moe_down": (I, [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, P, P]),
    "ink_add_rmsnorm": (I, [P, P, P, F, P, I, I, P]),
    "ink_short_conv": (I, [P, I, P, P, P, P, I, I, I, P]),
    "ink_decode_attention_workspace_bytes": (Z, [I, I, I, I]),
    "ink_decode_attention": (I, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, F, P, P, P, Z, P]),
    "ink_update_kv": (I, [P, P, P, P, P, I, I, I, I, I, P]),
    "ink_expert_gemm_scratch_bytes": (Z, [I]),
    "ink_expert_gemm": (I, [P, I, P, P, P, P, P, I, I, I, I, I, I, I, P, Z, P, P]),
    "ink_expert_reduce": (I, [P, P, P, P, P, I, I, I, I, I, P]),
    "ink_expert_gemm_tc_scratch_bytes": (Z, [I, I]),
    "ink_expert_gemm_tc": (I, [P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, P, Z, P, P]),
    "ink_moe_stack_layer_bytes": (Z, []),
    "ink_moe_stack_encode_banks": (I, [P, P, ctypes.c_uint64, P, ctypes.c_uint64, P, ctypes.c_uint64, P, ctypes.c_uint64, I, I, I]),
    "ink_moe_stack_scratch_bytes": (Z, [I, I, I, I, I, I]),
    "ink_moe_stack_trace_offset": (Z, [I, I, I, I, I, I]),
    "ink_moe_stack_decode": (I, [P, I, P, P, P, P, I, F, I, I, I, I, I, P, Z, P, P]),
    "ink_moe_stack_symmetric_bytes": (Z, [I, I, I]),
    "ink_moe_stack_decode_tp": (I, [P, I, P, P, P, P, I, F, I, I, I, I, I, P, Z, I, I, P, P, P]),
    "ink_moe_stack_set_wait_limit": (I, [ctypes.c_longlong]),
}


def exported_symbols() -> list[str]:
    return list(_SIGNATURES)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIBRARY.exists():
            raise RuntimeError(
                f"{LIBRARY} is missing: build it with `python {LIBRARY.parent / 'csrc' / 'build.py'}` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback for this path.")
        handle = ctypes.CDLL(str(LIBRARY))
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = restype, argtypes
        if handle.ink_abi_version() != ABI_VERSION:
            raise RuntimeError(f"{LIBRARY} has ABI {handle.ink_abi_version()}, expected {ABI_VERSION}: rebuild it")
        _lib = handle
    return _lib


def check(code: int) -> None:
    if code != 0:
        raise RuntimeError(f"inkling_b200: {lib().ink_last_error().decode()} (code {code})")


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("inkling_b200 kernels run on CUDA tensors only (no CPU path)")
