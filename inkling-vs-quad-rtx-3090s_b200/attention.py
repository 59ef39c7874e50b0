"""The decode step of the reference's attention module on this library's kernels.

`MyInklingAttention.forward` with a decoding cache (my_inkling/model.py:504-622) is: the fused QKVR projection,
RMS norm of the query heads, short convolution + RMS norm of the key, short convolution of the value, `update_kv`,
relative-position bias + mask + `scaled_dot_product_attention`, the output projection (and its all-reduce under
tensor parallelism). Here the two dense projections stay library GEMVs (`torch.nn.functional.linear`), everything
between them runs in this library: `ink_short_conv`, `ink_add_rmsnorm`, `ink_decode_attention` (which also stores
the token in the caches). The cache object is the reference's `MyInklingCache` (or anything with the same fields:
`layers[i].k_cache / v_cache / conv_caches[0 | 1].cache`, `position`, `pad_counts`).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .kernels import add_rmsnorm, decode_attention, short_conv
from .kernels.paired_all_reduce import all_reduce


class DecodeAttention(nn.Module):
    def __init__(self, qkvr_weight, o_weight, q_norm_weight, k_norm_weight, k_taps, v_taps, rel_proj, *, layer_idx: int,
                 heads: int, kv_heads: int, head_dim: int, d_rel: int, window: int = 0, log_scaling_n_floor=None,
                 log_scaling_alpha: float = 0.1, eps: float = 1e-6, group=None):
        """Weights as the reference module holds them after `fuse_projections`: qkvr_weight BF16
        [(h + 2 hk) c + h d_rel, d], o_weight BF16 [d, h c], norm weights BF16 [c], taps FP32 [hk c, 1, K],
        rel_proj BF16 [d_rel, rel_extent]. `window` > 0 for a sliding layer. `group`: the tensor-parallel process
        group whose ranks hold slices of the heads (the output projection's partial sums are all-reduced)."""
        super().__init__()
        self.layer_idx, self.heads, self.kv_heads, self.head_dim, self.d_rel = layer_idx, heads, kv_heads, head_dim, d_rel
        self.window, self.n_floor, self.alpha, self.eps, self.group = window, log_scaling_n_floor, log_scaling_alpha, eps, group
        self.sizes = [heads * head_dim, kv_heads * head_dim, kv_heads * head_dim, heads * d_rel]
        assert qkvr_weight.shape[0] == sum(self.sizes)
        for name, t in (("qkvr_weight", qkvr_weight), ("o_weight", o_weight), ("q_norm_weight", q_norm_weight),
                        ("k_norm_weight", k_norm_weight), ("k_taps", k_taps), ("v_taps", v_taps), ("rel_proj", rel_proj)):
            self.register_buffer(name, t.contiguous())
        self._zeros = None

    @classmethod
    def from_reference(cls, attention, group=None) -> "DecodeAttention":
        """From a `MyInklingAttention` whose projections are fused (`fuse_projections`), on its device."""
        return cls(attention.qkvr_proj.weight.detach(), attention.o_proj.weight.detach(), attention.q_norm.weight.detach(),
                   attention.k_norm.weight.detach(), attention.k_sconv.conv1d.weight.detach(),
                   attention.v_sconv.conv1d.weight.detach(), attention.rel_logits_proj.proj.detach(),
                   layer_idx=attention.layer_idx, heads=attention.num_heads, kv_heads=attention.num_key_value_heads,
                   head_dim=attention.head_dim, d_rel=attention.rel_logits_proj.d_rel, window=attention.sliding_window or 0,
                   log_scaling_n_floor=attention.log_scaling_n_floor, log_scaling_alpha=attention.log_scaling_alpha,
                   eps=attention.q_norm.variance_epsilon, group=group)

    def _norm(self, rows: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """RMS norm over the last dimension of BF16 [n, c] with the reference's rounding (kernels/decode.py:36-43)."""
        if self._zeros is None or self._zeros.shape[0] < rows.shape[0]:
            self._zeros = torch.zeros(rows.shape[0], rows.shape[1], dtype=torch.float32, device=rows.device)
        normed = torch.empty_like(rows)
        add_rmsnorm(self._zeros[: rows.shape[0]], rows, weight, self.eps, normed)   # rows + 0, then the norm
        return normed

    def forward(self, hidden_states: torch.Tensor, cache) -> torch.Tensor:
        """hidden_states BF16 [bs, 1, d], cache in decode mode -> BF16 [bs, 1, d]; the caches and the convolution
        histories of this layer are updated in place, `cache.position` is left to the caller (`cache.advance`)."""
        bs, s, _ = hidden_states.shape
        assert s == 1, "one token per sequence"
        layer = cache.layers[self.layer_idx]
        h, hk, c = self.heads, self.kv_heads, self.head_dim
        q, k, v, r = F.linear(hidden_states, self.qkvr_weight).split(self.sizes, dim=-1)
        q = self._norm(q.reshape(bs * h, c).contiguous(), self.q_norm_weight)
        k = short_conv(k.contiguous(), self.k_taps, layer.conv_caches[0].cache, None)
        k = self._norm(k.reshape(bs * hk, c), self.k_norm_weight)
        v = short_conv(v.contiguous(), self.v_taps, layer.conv_caches[1].cache, None)
        out = decode_attention(q.view(bs, h, c), r.reshape(bs, h, self.d_rel), self.rel_proj, layer.k_cache, layer.v_cache,
                               cache.position, cache.pad_counts, window=self.window, log_scaling_n_floor=self.n_floor,
                               log_scaling_alpha=self.alpha, scale=1.0 / c, new_key=k.view(bs, hk, 1, c),
                               new_value=v.reshape(bs, hk, 1, c))
        y = F.linear(out.reshape(bs, 1, h * c), self.o_weight)
        if self.group is not None:
            y = all_reduce(y, self.group)   # (nothing to do with one rank)
        return y


class DecodeLayer(nn.Module):
    """One sparse decoder layer at decode, `MyInklingDecoderLayer.forward` (my_inkling/model.py:661-675):
    h' = attn_sconv(attention(input_norm(h)), residual=h);  out = mlp_sconv(moe(post_norm(h')), residual=h').
    `attention` is a DecodeAttention, `moe` a FusedMoE (a sparse layer) or a DenseMLP (a dense one); the two short
    convolutions use the layer's convolution caches 2 and 3 of the reference's cache object."""

    def __init__(self, attention: DecodeAttention, moe, input_norm_weight, post_norm_weight, attn_taps, mlp_taps, eps: float = 1e-6):
        super().__init__()
        self.attention, self.moe, self.eps = attention, moe, eps
        for name, t in (("input_norm_weight", input_norm_weight), ("post_norm_weight", post_norm_weight),
                        ("attn_taps", attn_taps), ("mlp_taps", mlp_taps)):
            self.register_buffer(name, t.contiguous())
        self._zeros = None

    def _norm(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        rows = x.reshape(-1, x.shape[-1]).clone()          # (the norm kernel adds its FP32 input to the rows in place: zero here)
        if self._zeros is None or self._zeros.shape != rows.shape:
            self._zeros = torch.zeros(rows.shape, dtype=torch.float32, device=rows.device)
        normed = torch.empty_like(rows)
        add_rmsnorm(self._zeros, rows, weight, self.eps, normed)
        return normed.view(x.shape)

    def forward(self, hidden_states: torch.Tensor, cache) -> torch.Tensor:
        """hidden_states BF16 [bs, 1, d] -> BF16 [bs, 1, d]; the layer's caches are updated in place."""
        bs, _, d = hidden_states.shape
        layer = cache.layers[self.attention.layer_idx]
        attended = self.attention(self._norm(hidden_states, self.input_norm_weight), cache)
        h = short_conv(attended.contiguous(), self.attn_taps, layer.conv_caches[2].cache, hidden_states.contiguous())
        normed = self._norm(h, self.post_norm_weight).view(bs, d)
        block = self.moe.forward_partial(normed) if hasattr(self.moe, "forward_partial") else self.moe(normed)   # [bs, d], all-reduced
        return short_conv(block.view(bs, 1, d).contiguous(), self.mlp_taps, layer.conv_caches[3].cache, h)


class DenseMLP(nn.Module):
    """`MyInklingMLP` (my_inkling/model.py:153-171), the block of a dense layer: three library GEMVs,
    down(silu(gate(x)) * up(x)) * global_scale, BF16 like the reference's; all-reduced over `group` when the rows of
    gate/up and the columns of down are sliced."""

    def __init__(self, gate_weight, up_weight, down_weight, global_scale, group=None):
        super().__init__()
        for name, t in (("gate_weight", gate_weight), ("up_weight", up_weight), ("down_weight", down_weight), ("global_scale", global_scale)):
            self.register_buffer(name, t.contiguous())
        self.group = group

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = F.linear(F.silu(F.linear(x, self.gate_weight)) * F.linear(x, self.up_weight), self.down_weight) * self.global_scale
        return y if self.group is None else all_reduce(y, self.group)


class DecodeModel(nn.Module):
    """One decode step of the reference's model, `MyInkling.forward` with a decoding cache (my_inkling/model.py:679-800):
    normed embedding, the decoder layers, the final norm, the logits (hidden / mup multiplier through the LM head), and
    the cache's position counter moved on by one token."""

    def __init__(self, embedding, embed_norm_weight, layers, final_norm_weight, lm_head_weight, mup_multiplier: float,
                 eps: float = 1e-6, unpadded_vocab_size=None):
        super().__init__()
        for name, t in (("embedding", embedding), ("embed_norm_weight", embed_norm_weight), ("final_norm_weight", final_norm_weight),
                        ("lm_head_weight", lm_head_weight)):
            self.register_buffer(name, t.contiguous())
        self.layers = nn.ModuleList(layers)
        self.mup, self.eps, self.unpadded = float(mup_multiplier), eps, unpadded_vocab_size

    def forward(self, input_ids: torch.Tensor, cache) -> torch.Tensor:
        """input_ids int64 [bs, 1] -> logits BF16 [bs, 1, vocab]."""
        norm = self.layers[0]._norm
        hidden = norm(F.embedding(input_ids, self.embedding), self.embed_norm_weight)
        for layer in self.layers:
            hidden = layer(hidden, cache)
        hidden = norm(hidden, self.final_norm_weight) / self.mup
        logits = F.linear(hidden, self.lm_head_weight)
        cache.position.add_(1)
        return logits if self.unpadded is None else logits[..., : self.unpadded]
