"""CPU oracle (test infrastructure, never on the product path): the routed-expert
MoE layer of the reference, restated in plain torch on the CPU.

Every function names the reference lines it follows (paths are relative to the
reference project). Two yard-sticks are provided for the expert math:

* `*_reference`  -- keeps every BF16 rounding the reference performs, in the order
                    it performs them;
* `*_fp32`       -- the same weights and BF16 activations, float64 arithmetic and
                    no intermediate rounding: the yard-stick for the 2e-2 bar.

Pinning: the router, shared experts, unquantised expert loop and whole layer are
checked against fixtures produced by importing the reference's own classes; the
plan, grouped GEMM (NVFP4 dequant) and weighted reduce against its Triton kernels
run under the Triton interpreter; the per-route GEMV against its CUDA C file
compiled for the CPU behind an execution shim (tests/golden/make_golden.py).
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

from . import nvfp4

BF16 = torch.bfloat16


# --------------------------------------------------------------------- router
def router(x, weight, bias, global_scale, route_scale: float, top_k: int, n_shared: int):
    """my_inkling/model.py:311-350.

    x [t, d] (BF16 in production), weight [e_r + n_shared, d], bias FP32 [e_r],
    global_scale [1]. Returns (routed_logits [t, e_r], topk_weights [t, k],
    topk_indices int64 [t, k] (unsorted), shared_gammas [t, n_shared]).
    """
    logits = F.linear(x, weight)                                   # :326
    scores = logits.sigmoid()                                      # :328
    scores_for_choice = scores[..., :-n_shared] + bias             # :329-330 (FP32 bias => FP32)
    topk_indices = torch.topk(scores_for_choice, top_k, dim=-1, sorted=False)[1]  # :331-333
    routed_logits = logits[..., :-n_shared]
    shared_logits = logits[..., -n_shared:]
    topk_logits = torch.cat([routed_logits.gather(-1, topk_indices), shared_logits], dim=-1)
    log_probs = F.logsigmoid(topk_logits)                          # :340
    w = torch.exp(log_probs - torch.logsumexp(log_probs, dim=-1, keepdim=True))  # :341-343
    w = w * route_scale * global_scale                             # :345
    return routed_logits, w[..., :top_k].contiguous(), topk_indices, w[..., -n_shared:].contiguous()


def router_choice_scores(x, weight, bias, n_shared: int):
    """FP32 scores the top-k is taken over (model.py:326-330), for tie analysis."""
    logits = F.linear(x, weight)
    return logits.sigmoid()[..., :-n_shared] + bias


def router_fragile_tokens(x, weight, bias, n_shared: int, top_k: int, ulp_margin: float = 0.02):
    """Tokens whose top-k SET is not determined by exact arithmetic.

    A token is fragile when (a) its k-th and (k+1)-th scores are equal (torch.topk's
    tie-breaking is implementation defined), or (b) some expert that could cross the
    selection boundary has a float64 logit within `ulp_margin` BF16 ulps of a BF16
    rounding boundary (an FP32 dot product summed in another order may round the other
    way). Returns a bool tensor [t].
    """
    w64, x64 = weight.double(), x.double()
    logits64 = x64 @ w64.T
    scores = router_choice_scores(x, weight, bias, n_shared).double()
    ordered = scores.sort(dim=-1, descending=True).values
    kth, nxt = ordered[:, top_k - 1], ordered[:, top_k]
    tied = kth == nxt
    # (b): distance of the exact logit to the nearest BF16 rounding boundary
    routed = logits64[:, : scores.shape[1]]
    as_bf16 = routed.to(BF16).double()
    ulp = torch.maximum(as_bf16.abs(), torch.tensor(2.0**-126, dtype=torch.float64))
    ulp = 2.0 ** (torch.floor(torch.log2(ulp)) - 7)
    dist_to_boundary = (0.5 * ulp - (routed - as_bf16).abs()).abs() / ulp
    near = dist_to_boundary < ulp_margin
    # only experts whose score could reach the boundary matter
    s_up = (as_bf16 + ulp).to(BF16).sigmoid().double() + bias.double()
    s_dn = (as_bf16 - ulp).to(BF16).sigmoid().double() + bias.double()
    hi, lo = torch.maximum(s_up, s_dn), torch.minimum(s_up, s_dn)
    crosses = (hi >= kth[:, None]) & (lo <= kth[:, None]) | (hi >= nxt[:, None]) & (lo <= nxt[:, None])
    return tied | (near & crosses).any(-1)


# ----------------------------------------------------------------------- plan
def expert_plan(indices, sources, start: int, local: int, stride: int, capacity: int, max_expert: int | None = None):
    """kernels/expert_planner.py:44-56 (counts), :88-98 (compaction), :100-113
    (pointer table) with every expert resident (Resident == 1, SLOTS == 0), so the
    pointer of an active expert is its source address.

    indices: int64 [t, k]; sources: int64 [local, stride].
    Returns dict(experts int32 [local], counts int32 [local], rows int32
    [local, capacity] (-1 where the reference leaves memory untouched),
    pointers int64 [(max_expert+1)*stride]).
    """
    ids = np.asarray(indices).reshape(-1).astype(np.int64)
    sources = np.asarray(sources).astype(np.int64).reshape(local, stride)
    if max_expert is None:
        max_expert = start + local - 1
    experts = np.full(local, -1, np.int32)
    counts = np.zeros(local, np.int32)
    rows = np.full((local, capacity), -1, np.int32)
    pointers = np.zeros((max_expert + 1) * stride, np.int64)
    group = 0
    for e in range(local):
        routes = np.nonzero(ids == start + e)[0]          # ascending route numbers
        if routes.size == 0:
            continue
        experts[group] = start + e
        counts[group] = routes.size
        rows[group, : routes.size] = routes
        pointers[(start + e) * stride : (start + e + 1) * stride] = sources[e]
        group += 1
    return dict(experts=experts, counts=counts, rows=rows, pointers=pointers)


# ------------------------------------------------------------- routed experts
def _bf16_round(t: torch.Tensor) -> torch.Tensor:
    return t.to(BF16).to(t.dtype)


def routed_decode_reference(x, indices, weights, banks, max_expert: int | None = None):
    """kernels/routed_decode.cu:137-219 (gate_up then down_reduce), NVFP4 banks.

    x BF16 [t, d]; indices int64 [t, k]; weights BF16 [t, k];
    banks: {expert: {"gate_up_proj": u8 [2f, d/2], "gate_up_proj_scale": u8 [2f, d/16],
    "gate_up_proj_scale2": f32 [], "down_proj": u8 [d, f/2], "down_proj_scale",
    "down_proj_scale2"}}; experts absent from `banks` are skipped like a zero
    pointer row (:149,:199). Returns (activated BF16 [t*k, f], out FP32 [t, d]).

    Roundings kept: Y = bf16(silu(gate) * up) with gate/up FP32 (:169-171);
    per route bf16(bf16(dot * scale2) * w), summed in FP32 in choice order (:213-214).
    Dot products are float64 here (the kernel's FP32 summation order is not part of
    the contract).
    """
    t, d = x.shape
    k = indices.shape[1]
    any_bank = next(iter(banks.values()))
    f = any_bank["gate_up_proj"].shape[0] // 2
    if max_expert is None:
        max_expert = max(banks)
    x64 = x.double()
    activated = torch.zeros(t * k, f, dtype=BF16)
    out = torch.zeros(t, d, dtype=torch.float32)
    for token in range(t):
        total = torch.zeros(d, dtype=torch.float32)
        for choice in range(k):
            route = token * k + choice
            e = int(indices[token, choice])
            if e < 0 or e > max_expert or e not in banks:
                continue
            b = banks[e]
            values, block = nvfp4.decode_parts(b["gate_up_proj"], b["gate_up_proj_scale"])
            w_gu = values.double() * block.double().repeat_interleave(16, -1)
            s2 = torch.as_tensor(b["gate_up_proj_scale2"]).float().reshape(-1)[0]
            proj = (w_gu @ x64[token]).float() * s2                       # :167-168
            gate, up = proj[0::2], proj[1::2]                             # :162-166
            y = (gate / (1.0 + torch.exp(-gate)) * up).to(BF16)           # :169
            activated[route] = y
            values, block = nvfp4.decode_parts(b["down_proj"], b["down_proj_scale"])
            w_dn = values.double() * block.double().repeat_interleave(16, -1)
            s2 = torch.as_tensor(b["down_proj_scale2"]).float().reshape(-1)[0]
            down = _bf16_round((w_dn @ y.double()).float() * s2)          # :213
            total += _bf16_round(down * weights[token, choice].float())   # :214
        out[token] = total
    return activated, out


def routed_experts_dequant_reference(x, indices, weights, banks):
    """scripts/run_naive.py:86-108: dequantise each selected expert to BF16 on every
    forward, F.linear, de-interleave, silu*up, F.linear, scale by the router weight,
    index_add into a BF16 output. This is 'the reference's PyTorch NVFP4
    dequant+matmul path' and the timed CPU baseline."""
    out = torch.zeros_like(x)
    for e in torch.unique(indices).tolist():
        if e not in banks:
            continue
        b = banks[e]
        tokens, slots = torch.where(indices == e)
        w = nvfp4.dequant_bf16(b["gate_up_proj"], b["gate_up_proj_scale"], b["gate_up_proj_scale2"]).to(x.dtype)
        projected = F.linear(x[tokens], w)
        activated = F.silu(projected[:, 0::2]) * projected[:, 1::2]     # :103
        w = nvfp4.dequant_bf16(b["down_proj"], b["down_proj_scale"], b["down_proj_scale2"]).to(x.dtype)
        values = F.linear(activated, w)
        values = values * weights[tokens, slots, None]
        out.index_add_(0, tokens, values.to(x.dtype))
    return out


def routed_experts_fp32(x, indices, weights, banks):
    """Same inputs, float64 arithmetic, no intermediate rounding. Returns float64."""
    t, d = x.shape
    out = torch.zeros(t, d, dtype=torch.float64)
    cache = {}
    for token in range(t):
        for choice in range(indices.shape[1]):
            e = int(indices[token, choice])
            if e not in banks:
                continue
            if e not in cache:
                b = banks[e]
                cache[e] = (
                    nvfp4.dequant_exact(b["gate_up_proj"], b["gate_up_proj_scale"], b["gate_up_proj_scale2"]),
                    nvfp4.dequant_exact(b["down_proj"], b["down_proj_scale"], b["down_proj_scale2"]),
                )
            w_gu, w_dn = cache[e]
            proj = w_gu @ x[token].double()
            gate, up = proj[0::2], proj[1::2]
            out[token] += (w_dn @ (gate * torch.sigmoid(gate) * up)) * weights[token, choice].double()
    return out


# ------------------------------------------------------------- shared experts
def shared_experts_reference(x, gammas, gate_proj, up_proj, down_proj):
    """my_inkling/model.py:192-226 with torch ops in the input dtype: bmm gate, bmm up,
    silu(gate)*up*gamma, bmm down, FP32 sum over the shared experts, cast back.
    x [t, d]; gammas [t, e_s]; gate/up [e_s, f, d]; down [e_s, d, f]."""
    e_s = gate_proj.shape[0]
    h = x.unsqueeze(0).expand(e_s, -1, -1)
    g = gammas.T.unsqueeze(-1)
    gate = torch.bmm(h, gate_proj.transpose(1, 2))
    up = torch.bmm(h, up_proj.transpose(1, 2))
    activated = F.silu(gate) * up * g
    down = torch.bmm(activated, down_proj.transpose(1, 2))
    return down.float().sum(dim=0).to(x.dtype)


def shared_experts_fp32(x, gammas, gate_proj, up_proj, down_proj):
    x64 = x.double()
    out = torch.zeros(x.shape[0], down_proj.shape[1], dtype=torch.float64)
    for e in range(gate_proj.shape[0]):
        gate = x64 @ gate_proj[e].double().T
        up = x64 @ up_proj[e].double().T
        act = gate * torch.sigmoid(gate) * up * gammas[:, e : e + 1].double()
        out += act @ down_proj[e].double().T
    return out


# ---------------------------------------------------------------- whole layer
def moe_layer_reference(x, p, banks):
    """my_inkling/model.py:361-374: gate -> experts -> + shared experts, each in the
    dtype of x, with the routed experts taken through the dequantising path."""
    _, w, idx, gam = router(x, p["router_weight"], p["router_bias"], p["global_scale"],
                            p["route_scale"], p["top_k"], p["n_shared"])
    routed = routed_experts_dequant_reference(x, idx, w, banks)
    shared = shared_experts_reference(x, gam, p["shared_gate"], p["shared_up"], p["shared_down"])
    return routed + shared, idx, w, gam


def moe_layer_fp32(x, p, banks, indices, weights, gammas):
    """float64 layer output for GIVEN routing (indices/weights/gammas as produced by
    the implementation under test), so that only expert arithmetic is compared."""
    return routed_experts_fp32(x, indices, weights, banks) + shared_experts_fp32(
        x, gammas, p["shared_gate"], p["shared_up"], p["shared_down"])


# -------------------------------------------------------------- grouped path
def expert_gemm_reference(x, plan, banks, projection: int, top_k: int, n: int, capacity_rows: int):
    """kernels/grouped_experts.py:26-148. Returns [capacity_rows, n or n/2] in the
    dtype of x; rows not written stay zero. Weight tile = dtype(E2M1*(E4M3*scale2))
    (:118), FP32 accumulate of the products (:126) -- float64 here -- then SwiGLU on
    the de-interleaved pairs for projection 0 (:128-138)."""
    name = "gate_up_proj" if projection == 0 else "down_proj"
    width = n // 2 if projection == 0 else n
    y = torch.zeros(capacity_rows, width, dtype=x.dtype)
    for g, e in enumerate(plan["experts"]):
        if e < 0:
            break
        b = banks[int(e)]
        w = nvfp4.dequant_as(b[name], b[name + "_scale"], b[name + "_scale2"], x.dtype).double()
        for route in plan["rows"][g, : plan["counts"][g]]:
            route = int(route)
            row = route // top_k if projection == 0 else route
            acc = w @ x[row].double()
            if projection == 0:
                gate, up = acc[0::2].float(), acc[1::2].float()
                y[route] = (gate * torch.sigmoid(gate) * up).to(x.dtype)
            else:
                y[route] = acc.float().to(x.dtype)
    return y


def expert_reduce_reference(down, indices, weights, active, output):
    """kernels/grouped_experts.py:152-186: output[token] += sum over choices of
    fp32(bf16(down[route] * w)), skipping inactive routes. `active` bool [t, k]."""
    t, k = indices.shape
    out = output.clone()
    for token in range(t):
        acc = torch.zeros(down.shape[1], dtype=torch.float32)
        for choice in range(k):
            route = token * k + choice
            value = down[route].float() if bool(active[token, choice]) else torch.zeros(down.shape[1])
            acc += (value * weights[token, choice].float()).to(down.dtype).float()
        out[token] += acc
    return out


# ----------------------------------------------------------------- TP slices
def shard_banks(bank: dict, rank: int, world: int) -> dict:
    """scripts/make_flashpack.py:30-35,83-95: gate_up banks are cut on rows (dim 0 of
    one expert's [2f, ...] tensors: a contiguous run of interleaved rows), down banks
    on packed columns; `_scale2` is replicated."""
    out = {}
    for name, tensor in bank.items():
        if name in ("gate_up_proj", "gate_up_proj_scale"):
            size = tensor.shape[0] // world
            out[name] = tensor[rank * size : (rank + 1) * size].contiguous()
        elif name in ("down_proj", "down_proj_scale"):
            size = tensor.shape[1] // world
            out[name] = tensor[:, rank * size : (rank + 1) * size].contiguous()
        else:
            out[name] = tensor
    return out


def shard_shared(gate_proj, up_proj, down_proj, rank: int, world: int):
    """my_inkling/tp_plan.py:139-140: gate/up on dim 1, down on dim 2."""
    f = gate_proj.shape[1] // world
    sl = slice(rank * f, (rank + 1) * f)
    return gate_proj[:, sl].contiguous(), up_proj[:, sl].contiguous(), down_proj[:, :, sl].contiguous()


# ---------------------------------------------------------------- BF16 experts
def routed_decode_bf16_reference(x, indices, weights, banks, max_expert: int | None = None):
    """kernels/routed_decode.cu:137-219 compiled with QUANT=0 (row_dot :85-101): BF16
    weight banks, pointer stride 2 (kernels/grouped_experts.py:9-22 with
    quantized=False), no scales. banks: {expert: {"gate_up_proj": BF16 [2f, d] (rows
    interleave gate and up), "down_proj": BF16 [d, f]}}. Same roundings as the
    NVFP4 kernels with scale 1: Y = bf16(silu(gate) * up); per route
    bf16(bf16(dot) * w), FP32 sum in choice order. Dot products are float64 here.
    Returns (activated BF16 [t*k, f], out FP32 [t, d])."""
    t, d = x.shape
    k = indices.shape[1]
    f = next(iter(banks.values()))["gate_up_proj"].shape[0] // 2
    if max_expert is None:
        max_expert = max(banks)
    activated = torch.zeros(t * k, f, dtype=BF16)
    out = torch.zeros(t, d, dtype=torch.float32)
    for token in range(t):
        total = torch.zeros(d, dtype=torch.float32)
        for choice in range(k):
            e = int(indices[token, choice])
            if e < 0 or e > max_expert or e not in banks:
                continue
            proj = (banks[e]["gate_up_proj"].double() @ x[token].double()).float()
            gate, up = proj[0::2], proj[1::2]
            y = (gate / (1.0 + torch.exp(-gate)) * up).to(BF16)
            activated[token * k + choice] = y
            down = _bf16_round((banks[e]["down_proj"].double() @ y.double()).float())
            total += _bf16_round(down * weights[token, choice].float())
        out[token] = total
    return activated, out


def routed_experts_bf16_fp32(x, indices, weights, banks):
    """The BF16-expert layer in float64 with no intermediate rounding."""
    out = torch.zeros(x.shape[0], x.shape[1], dtype=torch.float64)
    for token in range(x.shape[0]):
        for choice in range(indices.shape[1]):
            e = int(indices[token, choice])
            if e not in banks:
                continue
            proj = banks[e]["gate_up_proj"].double() @ x[token].double()
            gate, up = proj[0::2], proj[1::2]
            out[token] += (banks[e]["down_proj"].double() @ (gate * torch.sigmoid(gate) * up)) * weights[token, choice].double()
    return out


# ------------------------------------------------------------------ layer glue
def rms_norm_reference(x, weight, eps: float):
    """my_inkling/model.py:143-150 (the CPU branch of MyInklingRMSNorm.forward) and its
    Triton twin kernels/decode.py:36-43: FP32 mean of squares, x * rsqrt(var + eps), the
    normalised value rounded to the input dtype BEFORE the multiplication by the weight,
    product in the input dtype."""
    input_dtype = x.dtype
    h = x.float()
    variance = h.pow(2).mean(-1, keepdim=True)
    h = h * torch.rsqrt(variance + eps)
    return weight.to(input_dtype) * h.to(input_dtype)


def add_rms_norm_reference(partial, residual, weight, eps: float):
    """The skeleton of my_inkling/model.py:672-675 for a stack of MoE blocks: the block's
    FP32 output is cast to BF16 (my_inkling/offloaded_experts.py:314) and added to the
    BF16 residual stream (a BF16 tensor add), then normalised for the next block.
    Returns (new residual BF16, normed BF16)."""
    new_residual = residual + partial.to(residual.dtype)
    return new_residual, rms_norm_reference(new_residual, weight, eps)


def short_conv_reference(x, weight, history, residual=None):
    """kernels/decode.py:65-112 (_short_conv, one new token against its cached history):
    per channel total = sum_j history[j + 1] * w[j] (j < K - 1) + x * w[K - 1] in FP32,
    history shifted by one with x appended (FP32), output = dtype(total + x), and with a
    residual: dtype(fp32(output) + residual). x [bs, d]; weight [d, K] (the conv1d weight
    [d, 1, K] squeezed); history FP32 [bs, d, K]. Returns (y, new_history)."""
    k = weight.shape[-1]
    current = x.float()
    w = weight.float()
    total = torch.zeros_like(current)
    new_history = history.clone()
    for j in range(k - 1):
        previous = history[..., j + 1]
        total = total + previous * w[:, j]
        new_history[..., j] = previous
    total = total + current * w[:, k - 1]
    new_history[..., k - 1] = current
    y = (total + current).to(x.dtype)
    if residual is not None:
        y = (y.float() + residual.float()).to(x.dtype)
    return y, new_history


def stack_reference(x, blocks, norm_weight, eps: float):
    """A stack of MoE blocks joined the way configs with several blocks join them:
    n_0 = x (taken as already normalised), h_0 = x; per block m = moe(n) through the
    reference-faithful BF16 layer (moe_layer_reference), h += m, n = rms_norm(h).
    `blocks` is a list of (p, banks). Returns dict(normed, residual, routing=[idx per
    block], moe_out=[per block])."""
    h, n = x.clone(), x.clone()
    routing, outs = [], []
    for p, banks in blocks:
        m, idx, _, _ = moe_layer_reference(n, p, banks)
        h = h + m
        n = rms_norm_reference(h, norm_weight, eps)
        routing.append(idx)
        outs.append(m)
    return dict(normed=n, residual=h, routing=routing, moe_out=outs)


def stack_fp32(x, blocks, norm_weight, eps: float, routing):
    """The same stack with the expert arithmetic of every block in float64 (no
    intermediate rounding inside a block) for GIVEN routing -- `routing[i]` =
    (indices, weights, gammas) of block i as the implementation under test chose them --
    and the roundings the glue performs between blocks (BF16 block output, BF16 add,
    RMS norm as rms_norm_reference). Returns (normed BF16, residual BF16)."""
    h, n = x.clone(), x.clone()
    for (p, banks), (idx, w, gam) in zip(blocks, routing):
        m = moe_layer_fp32(n, p, banks, idx, w, gam).float()
        h, n = add_rms_norm_reference(m, h, norm_weight, eps)
    return n, h
