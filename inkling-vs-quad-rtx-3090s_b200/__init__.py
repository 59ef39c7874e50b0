"""B200 (sm_100a) NVFP4 routed-expert path for the Inkling-Small MoE engine."""
from . import kernels
from .attention import DecodeAttention, DecodeLayer, DecodeModel, DenseMLP
from .layer import (MATVEC_TOKENS, FusedMoE, ResidentExperts, apply_fused_moe_plan, apply_resident_plan)
from .stack import DecodeStackGraph, MoEStack
from .synthetic import ExpertBanks, make_expert_banks, make_layer_params, quantize_nvfp4

__all__ = [
    "DecodeAttention", "DecodeLayer", "DecodeModel", "DecodeStackGraph", "DenseMLP", "ExpertBanks", "FusedMoE", "MoEStack", "MATVEC_TOKENS", "ResidentExperts", "apply_fused_moe_plan",
    "apply_resident_plan", "kernels", "make_expert_banks", "make_layer_params", "quantize_nvfp4",
]
