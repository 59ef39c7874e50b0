"""Decode attention with the relative-position bias, and the cache update in front of it.

`update_kv` keeps the reference's call (kernels/decode.py:199-230) for the decode step; `decode_attention` is
the part of `MyInklingAttention.forward` (my_inkling/model.py:533-612, `static_decode`) between the normed query
and the output projection, which the reference runs as `rel_logits_proj` + mask + `scaled_dot_product_attention`.
"""
from __future__ import annotations

import torch

from . import _abi

_workspaces: dict = {}   # (device, bytes) -> buffer for the partial results, reused from call to call (one stream)


def update_kv(key, value, k_cache, v_cache, start, window: int = 0) -> None:
    """key, value BF16 [bs, hk, 1, c] (any strides over bs/hk, as the reference's transposed views), caches BF16
    [bs, hk, capacity, c] contiguous, `start` the device int64 position counter (decode). Stores the token at slot
    start (modulo `window` in a sliding layer)."""
    bs, hk, s, c = key.shape
    assert s == 1, "decode stores one token per step"
    assert isinstance(start, torch.Tensor) and start.dtype == torch.int64, "decode counts on the device"
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape == v_cache.shape
    assert k_cache.shape[0] == bs and k_cache.shape[1] == hk and k_cache.shape[3] == c
    new_k = key.reshape(bs, hk, c).contiguous()
    new_v = value.reshape(bs, hk, c).contiguous()
    _abi.require_cuda(new_k, new_v, k_cache, v_cache, start)
    _abi.check(_abi.lib().ink_update_kv(new_k.data_ptr(), new_v.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                        start.data_ptr(), bs, hk, c, k_cache.shape[2], int(window), _abi.stream()))


def decode_attention(query, relative_states, proj, k_cache, v_cache, position, pad_counts=None, *, window: int = 0,
                     log_scaling_n_floor=None, log_scaling_alpha: float = 0.1, scale: float | None = None, out=None,
                     new_key=None, new_value=None):
    """query BF16 [bs, h, 1, c] or [bs, h, c] (after q_norm), relative_states BF16 [bs, 1, h, d_rel] or [bs, h, d_rel],
    proj BF16 [d_rel, rel_extent] (`rel_logits_proj.proj`), caches BF16 [bs, hk, slots, c] holding the current token,
    position the device int64 counter, pad_counts int64 [bs] or None -> BF16 [bs, h, 1, c] (what the reference's
    `scaled_dot_product_attention` call returns). `window` > 0: sliding layer (ring); else full attention, scaled
    logarithmically when `log_scaling_n_floor` is set. `scale` defaults to 1 / head_dim (my_inkling/model.py:448).
    With `new_key` / `new_value` BF16 [bs, hk, 1, c] the caches need not hold the current token yet: the call uses them
    for its slot and stores them there (the reference's `update_kv` + attention in one launch)."""
    bs, h = query.shape[0], query.shape[1]
    c = query.shape[-1]
    q = query.reshape(bs, h, c).contiguous()
    r = relative_states.reshape(bs, h, -1).contiguous()
    d_rel, extent = proj.shape
    assert r.shape[-1] == d_rel and proj.is_contiguous()
    assert q.dtype == r.dtype == proj.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape == v_cache.shape
    hk, slots = k_cache.shape[1], k_cache.shape[2]
    assert k_cache.shape[0] == bs and k_cache.shape[3] == c
    assert isinstance(position, torch.Tensor) and position.dtype == torch.int64
    if pad_counts is not None:
        assert pad_counts.dtype == torch.int64 and pad_counts.numel() == bs and pad_counts.is_contiguous()
    new_k = new_v = None
    if new_key is not None:
        new_k = new_key.reshape(bs, hk, c).contiguous()
        new_v = new_value.reshape(bs, hk, c).contiguous()
        assert new_k.dtype == new_v.dtype == torch.bfloat16
    if out is None:
        out = torch.empty((bs, h, 1, c), dtype=torch.bfloat16, device=q.device)
    need = _abi.lib().ink_decode_attention_workspace_bytes(bs, h, c, slots)
    workspace = None
    if need:
        key = (q.device, need)
        workspace = _workspaces.get(key)
        if workspace is None:
            workspace = _workspaces[key] = torch.zeros(need, dtype=torch.uint8, device=q.device)   # arrival counters start at zero
    _abi.require_cuda(q, r, proj, k_cache, v_cache, position, pad_counts, out, new_k, new_v)
    _abi.check(_abi.lib().ink_decode_attention(
        q.data_ptr(), r.data_ptr(), proj.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), position.data_ptr(),
        _abi.ptr(pad_counts), out.data_ptr(), bs, h, hk, c, d_rel, extent, slots, int(window),
        int(log_scaling_n_floor or 0), float(log_scaling_alpha), float(scale if scale is not None else 1.0 / c),
        _abi.ptr(new_k), _abi.ptr(new_v), _abi.ptr(workspace), need, _abi.stream()))
    return out
