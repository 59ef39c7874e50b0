"""Fused router (and router + plan) launches; see include/inkling_b200.h."""
from __future__ import annotations

import torch

from . import _abi


def router_workspace(tokens: int, n_experts_total: int, device) -> torch.Tensor:
    """Zero-filled scratch for `router_forward`; reusable across calls on one stream."""
    size = _abi.lib().ink_router_workspace_bytes(tokens, n_experts_total)
    return torch.zeros(size, dtype=torch.uint8, device=device)


def _common(x, weight, bias, global_scale, top_k, n_shared, topk_weights, topk_indices, shared_gammas, workspace):
    tokens, hidden = x.shape
    n_routed = weight.shape[0] - n_shared
    assert x.dtype == weight.dtype == global_scale.dtype == torch.bfloat16 and bias.dtype == torch.float32
    assert topk_weights.dtype == shared_gammas.dtype == torch.bfloat16 and topk_indices.dtype == torch.int64
    assert weight.shape[1] == hidden and bias.shape == (n_routed,)
    assert topk_weights.shape == topk_indices.shape == (tokens, top_k) and shared_gammas.shape == (tokens, n_shared)
    tensors = (x, weight, bias, global_scale, topk_weights, topk_indices, shared_gammas, workspace)
    assert all(t.is_contiguous() for t in tensors)
    _abi.require_cuda(*tensors)
    return tokens, hidden, n_routed


def router_forward(x, weight, bias, global_scale, route_scale: float, top_k: int, n_shared: int,
                   topk_weights, topk_indices, shared_gammas, workspace, routed_logits=None) -> None:
    tokens, hidden, n_routed = _common(x, weight, bias, global_scale, top_k, n_shared, topk_weights,
                                       topk_indices, shared_gammas, workspace)
    _abi.check(_abi.lib().ink_router_forward(
        x.data_ptr(), weight.data_ptr(), bias.data_ptr(), global_scale.data_ptr(), float(route_scale), tokens,
        hidden, n_routed, n_shared, top_k, _abi.ptr(routed_logits), topk_weights.data_ptr(),
        topk_indices.data_ptr(), shared_gammas.data_ptr(), workspace.data_ptr(), workspace.numel(), _abi.stream()))


def router_plan_forward(x, weight, bias, global_scale, route_scale: float, top_k: int, n_shared: int,
                        topk_weights, topk_indices, shared_gammas, workspace, sources, pointers, experts,
                        counts, rows, start: int, local: int, stride: int, capacity: int,
                        routed_logits=None) -> None:
    tokens, hidden, n_routed = _common(x, weight, bias, global_scale, top_k, n_shared, topk_weights,
                                       topk_indices, shared_gammas, workspace)
    _abi.require_cuda(sources, pointers, experts, counts, rows)
    _abi.check(_abi.lib().ink_router_plan_forward(
        x.data_ptr(), weight.data_ptr(), bias.data_ptr(), global_scale.data_ptr(), float(route_scale), tokens,
        hidden, n_routed, n_shared, top_k, _abi.ptr(routed_logits), topk_weights.data_ptr(),
        topk_indices.data_ptr(), shared_gammas.data_ptr(), workspace.data_ptr(), workspace.numel(),
        sources.data_ptr(), pointers.data_ptr(), experts.data_ptr(), counts.data_ptr(), rows.data_ptr(),
        start, local, stride, capacity, _abi.stream()))


def router_forward_static(x, weight, bias, global_scale, route_scale: float, top_k: int, n_shared: int,
                          topk_weights, topk_indices, shared_gammas, routed_logits=None) -> None:
    """`router_forward` without a workspace argument, for callers that may not allocate
    device memory: the kernel's scratch is an array inside the library (at most 8 tokens
    and 544 router rows). Calls share that array, so keep them on one stream; make the
    first call on a device outside graph capture (it looks the array's address up)."""
    workspace = topk_weights   # only to satisfy the shared argument checks; not passed on
    tokens, hidden, n_routed = _common(x, weight, bias, global_scale, top_k, n_shared, topk_weights,
                                       topk_indices, shared_gammas, workspace)
    _abi.check(_abi.lib().ink_router_forward_static(
        x.data_ptr(), weight.data_ptr(), bias.data_ptr(), global_scale.data_ptr(), float(route_scale), tokens,
        hidden, n_routed, n_shared, top_k, _abi.ptr(routed_logits), topk_weights.data_ptr(),
        topk_indices.data_ptr(), shared_gammas.data_ptr(), _abi.stream()))
