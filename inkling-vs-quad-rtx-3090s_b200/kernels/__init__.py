"""Drop-in counterpart of the reference's `kernels` package for the NVFP4
routed-expert path: same names, same call signatures, sm_100a library underneath."""
from .expert_planner import expert_copy, expert_plan
from .grouped_experts import block_scaled_supported, encode_bank_maps, expert_bank_names, expert_gemm, expert_reduce
from .attention import decode_attention, update_kv
from .routed_decode import add_rmsnorm, moe_decode, routed_decode, short_conv
from .stack import StackDescriptor, set_wait_limit, stack_supported
from .router import router_forward, router_forward_static, router_plan_forward, router_workspace

__all__ = [
    "add_rmsnorm",
    "block_scaled_supported",
    "encode_bank_maps",
    "expert_bank_names",
    "expert_copy",
    "expert_gemm",
    "expert_reduce",
    "expert_plan",
    "moe_decode",
    "routed_decode",
    "StackDescriptor",
    "set_wait_limit",
    "short_conv",
    "decode_attention",
    "update_kv",
    "stack_supported",
    "router_forward",
    "router_forward_static",
    "router_plan_forward",
    "router_workspace",
]
