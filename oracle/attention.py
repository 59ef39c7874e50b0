"""CPU restatement of the reference's decode attention (one query token per sequence). Test infrastructure:
only tests/, the smoke test and the bench's CPU legs may use this package.

Follows my_inkling/model.py:504-622 (`MyInklingAttention.forward`, the `static_decode` branch),
my_inkling/model.py:94-133 (`MyInklingRelativeLogits`), my_inkling/cache.py:213-228 (`decode_distance`) and
kernels/decode.py:149-196 (`_update_kv`). Pinned by tests/golden/attention.npz, which was produced by running those
modules (tests/golden/make_attention_golden.py).
"""
from __future__ import annotations

import math

import torch

BF16 = torch.bfloat16


def decode_distance(position: int, capacity: int, window: int) -> torch.Tensor:
    """cache.py:213-228: distance of every cache slot from the current token; a sliding layer's slots form a
    ring, so the distance is taken modulo the window (non-negative, Python remainder)."""
    distance = position - torch.arange(capacity)
    return distance.remainder(window) if window else distance


def relative_bias(r: torch.Tensor, proj: torch.Tensor, distance: torch.Tensor) -> torch.Tensor:
    """model.py:112-133: r BF16 [bs, h, d_rel] @ proj BF16 [d_rel, extent] (a BF16 matmul: FP32 sums rounded to
    BF16), gathered at the clamped distance, zero outside [0, extent). -> BF16 [bs, h, slots]"""
    extent = proj.shape[1]
    logits = (r.float() @ proj.float()).to(BF16)
    bias = logits[..., distance.clamp(0, extent - 1)]
    return bias.masked_fill((distance < 0) | (distance >= extent), 0.0)


def log_scaling_tau(position: int, n_floor, alpha: float) -> float | None:
    """model.py:583-590: 1 + alpha * log(max((position + 1) / n_floor, 1)) in FP32."""
    if not n_floor:
        return None
    ratio = torch.tensor((position + 1) / n_floor, dtype=torch.float32).clamp(min=1.0)
    return float(1.0 + alpha * torch.log(ratio))


def decode_attention(q, r, proj, k_cache, v_cache, position: int, pad_counts, window: int, n_floor, alpha: float,
                     scale: float, exact: bool = False) -> torch.Tensor:
    """q BF16 [bs, h, c] (after q_norm), r BF16 [bs, h, d_rel], caches BF16 [bs, hk, slots, c] with the current token
    already stored -> [bs, h, c]. `exact=False` keeps the module's BF16 roundings (the bias, the scaled query and
    the scaled mask) and rounds the result to BF16; `exact=True` does the same arithmetic in float64 without them."""
    bs, h, c = q.shape
    hk, slots = k_cache.shape[1], k_cache.shape[2]
    distance = decode_distance(position, slots, window)
    real = torch.float64 if exact else torch.float32
    if exact:
        extent = proj.shape[1]
        logits = r.double() @ proj.double()
        bias = logits[..., distance.clamp(0, extent - 1)].masked_fill((distance < 0) | (distance >= extent), 0.0)
    else:
        bias = relative_bias(r, proj, distance)
    allowed = (distance >= 0)[None, :] & (distance[None, :] <= (position - pad_counts.view(-1, 1)))   # model.py:551
    mask = bias.to(real).masked_fill(~allowed[:, None, :], float("-inf"))
    query = q.to(real)
    tau = None if window else log_scaling_tau(position, n_floor, alpha)     # full-attention layers only, model.py:578-590
    if tau is not None:
        query, mask = query * tau, mask * tau
        if not exact:
            query, mask = query.to(BF16).to(real), mask.to(BF16).to(real)
    group = h // hk
    keys = k_cache.to(real).repeat_interleave(group, dim=1)      # [bs, h, slots, c]
    values = v_cache.to(real).repeat_interleave(group, dim=1)
    scores = torch.einsum("bhc,bhsc->bhs", query, keys) * scale + mask
    weights = torch.softmax(scores, dim=-1)
    result = torch.einsum("bhs,bhsc->bhc", weights, values)
    return result if exact else result.to(BF16)


def update_kv(k_cache, v_cache, new_k, new_v, position: int, window: int) -> None:
    """kernels/decode.py:149-196 with one new token: store it at slot `position` (modulo the window in a sliding
    layer), in place."""
    slot = position % window if window else position
    k_cache[:, :, slot] = new_k
    v_cache[:, :, slot] = new_v


def rms_norm_heads(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """MyInklingRMSNorm over the last dimension (my_inkling/model.py:143-150): FP32 statistics, the normalised value
    rounded to the input type, then times the weight."""
    xf = x.float()
    normed = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
    return weight * normed


def short_conv_step(x: torch.Tensor, taps: torch.Tensor, history: torch.Tensor, residual=None) -> torch.Tensor:
    """One decode token through MyInklingShortConv (kernels/decode.py:65-146): x BF16 [bs, d], taps FP32 [d, 1, K],
    history FP32 [bs, d, K] shifted in place. total = sum_j history[j + 1] * taps[j] + x * taps[K - 1] in FP32, tap
    order; y = bf16(total + x), with a residual y = bf16(fp32(y) + residual)."""
    k = taps.shape[-1]
    w = taps[:, 0]                                   # [d, K]
    xf = x.float()
    total = torch.zeros_like(xf)
    for j in range(k - 1):
        total = total + history[:, :, j + 1] * w[:, j]
    total = total + xf * w[:, k - 1]
    history[:, :, :-1] = history[:, :, 1:].clone()
    history[:, :, -1] = xf
    y = (total + xf).to(BF16)
    return y if residual is None else (y.float() + residual.float()).to(BF16)


def attention_decode_step(hidden, weights: dict, k_cache, v_cache, k_history, v_history, position: int, pad_counts, *,
                          heads: int, kv_heads: int, head_dim: int, d_rel: int, window: int, n_floor, alpha: float,
                          eps: float) -> torch.Tensor:
    """`MyInklingAttention.forward` with a decoding cache (my_inkling/model.py:504-622), hidden BF16 [bs, d] -> BF16
    [bs, d]; caches and histories are updated in place. `weights`: qkvr [(h + 2 hk) c + h d_rel, d], o [d, h c],
    q_norm, k_norm [c], k_taps, v_taps FP32 [hk c, 1, K], rel_proj [d_rel, extent]."""
    bs = hidden.shape[0]
    h, hk, c = heads, kv_heads, head_dim
    qkvr = (hidden.float() @ weights["qkvr"].float().T).to(BF16)
    q, k, v, r = qkvr.split([h * c, hk * c, hk * c, h * d_rel], dim=-1)
    q = rms_norm_heads(q.reshape(bs, h, c), weights["q_norm"], eps)
    k = rms_norm_heads(short_conv_step(k, weights["k_taps"], k_history).reshape(bs, hk, c), weights["k_norm"], eps)
    v = short_conv_step(v, weights["v_taps"], v_history).reshape(bs, hk, c)
    update_kv(k_cache, v_cache, k, v, position, window)
    out = decode_attention(q, r.reshape(bs, h, d_rel), weights["rel_proj"], k_cache, v_cache, position, pad_counts, window,
                           n_floor, alpha, 1.0 / c)
    return (out.reshape(bs, h * c).float() @ weights["o"].float().T).to(BF16)
