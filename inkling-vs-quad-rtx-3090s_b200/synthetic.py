"""Seeded synthetic NVFP4 layers (the checkpoint and its tokenizer are not available
offline): weights N(0, std) quantised to the checkpoint's NVFP4 layout, built on the
device they will live on, expert by expert, so peak memory stays close to the final
footprint.
"""
from __future__ import annotations

import torch

BF16 = torch.bfloat16
_THRESHOLDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def quantize_nvfp4(weight: torch.Tensor):
    """FP32 [..., rows, K] -> (codes uint8 [..., rows, K/2], scales uint8 (E4M3 bytes)
    [..., rows, K/16], scale2 FP32 [...]). One scale2 per leading index (per bank):
    scale2 = amax/(6*448); block scale = e4m3(block amax/(6*scale2)); code = nearest E2M1
    of w/(scale*scale2); low nibble = even column."""
    w = weight.float()
    *lead, rows, k = w.shape
    assert k % 16 == 0
    amax = w.abs().amax(dim=(-2, -1), keepdim=True).clamp_min(1e-30)
    scale2 = amax / (6.0 * 448.0)
    blocks = w.view(*lead, rows, k // 16, 16)
    scale_f8 = (blocks.abs().amax(-1) / (6.0 * scale2)).clamp(max=448.0).to(torch.float8_e4m3fn)
    decoded = (scale_f8.float() * scale2).clamp_min(1e-30).unsqueeze(-1)
    ratio = blocks / decoded
    thresholds = torch.tensor(_THRESHOLDS, device=w.device)
    code = torch.bucketize(ratio.abs(), thresholds, out_int32=True) | ((ratio < 0).to(torch.int32) << 3)
    code = code.view(*lead, rows, k).to(torch.uint8)
    packed = code[..., 0::2] | (code[..., 1::2] << 4)
    return packed.contiguous(), scale_f8.view(torch.uint8).contiguous(), scale2.reshape(lead).float()


class ExpertBanks:
    """All NVFP4 experts of one layer (one rank's slice) in six contiguous device
    allocations, one per bank kind; `weights` exposes them per expert in the dictionary
    form the reference's expert runtime takes (my_inkling/offloaded_experts.py:41-53)."""

    def __init__(self, experts: int, hidden: int, intermediate: int, device):
        u8 = dict(dtype=torch.uint8, device=device)
        self.experts, self.hidden, self.intermediate = experts, hidden, intermediate
        self.gate_up_proj = torch.empty(experts, 2 * intermediate, hidden // 2, **u8)
        self.gate_up_proj_scale = torch.empty(experts, 2 * intermediate, hidden // 16, **u8)
        self.gate_up_proj_scale2 = torch.empty(experts, dtype=torch.float32, device=device)
        self.down_proj = torch.empty(experts, hidden, intermediate // 2, **u8)
        self.down_proj_scale = torch.empty(experts, hidden, intermediate // 16, **u8)
        self.down_proj_scale2 = torch.empty(experts, dtype=torch.float32, device=device)

    @property
    def weights(self) -> dict[int, dict[str, torch.Tensor]]:
        names = ("gate_up_proj", "gate_up_proj_scale", "gate_up_proj_scale2",
                 "down_proj", "down_proj_scale", "down_proj_scale2")
        return {e: {n: getattr(self, n)[e] for n in names} for e in range(self.experts)}

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (
            self.gate_up_proj, self.gate_up_proj_scale, self.gate_up_proj_scale2,
            self.down_proj, self.down_proj_scale, self.down_proj_scale2))


def make_expert_banks(experts: int, hidden: int, intermediate_full: int, device, seed: int, std: float = 0.02,
                      rank: int = 0, world: int = 1, chunk: int = 8) -> ExpertBanks:
    """Rank `rank`'s tensor-parallel slice of `experts` seeded experts: the full expert is
    generated and quantised, then sliced the way the reference shards the checkpoint
    (scripts/make_flashpack.py:30-35: gate_up on rows, down on packed columns, scale2
    replicated), so every rank holds a slice of the SAME weights. `chunk` experts are
    generated at a time to bound the temporaries."""
    f = intermediate_full // world
    banks = ExpertBanks(experts, hidden, f, device)
    gen = torch.Generator(device=device).manual_seed(seed)
    rows = slice(rank * 2 * f, (rank + 1) * 2 * f)
    for e0 in range(0, experts, chunk):
        n = min(chunk, experts - e0)
        gate_up = torch.randn(n, 2 * intermediate_full, hidden, generator=gen, device=device) * std
        codes, scales, scale2 = quantize_nvfp4(gate_up)
        banks.gate_up_proj[e0:e0 + n] = codes[:, rows]
        banks.gate_up_proj_scale[e0:e0 + n] = scales[:, rows]
        banks.gate_up_proj_scale2[e0:e0 + n] = scale2
        del gate_up, codes, scales
        down = torch.randn(n, hidden, intermediate_full, generator=gen, device=device) * std
        codes, scales, scale2 = quantize_nvfp4(down)
        banks.down_proj[e0:e0 + n] = codes[:, :, rank * f // 2:(rank + 1) * f // 2]
        banks.down_proj_scale[e0:e0 + n] = scales[:, :, rank * f // 16:(rank + 1) * f // 16]
        banks.down_proj_scale2[e0:e0 + n] = scale2
        del down, codes, scales
    return banks


def make_layer_params(hidden: int, intermediate_full: int, experts: int, n_shared: int, device, seed: int,
                      std: float = 0.02, rank: int = 0, world: int = 1, bias_std: float = 0.0) -> dict:
    """Router (replicated) and shared experts (sliced on the FFN width, reference:
    my_inkling/tp_plan.py:139-140) for one layer."""
    gen = torch.Generator(device=device).manual_seed(seed + 7919)
    f = intermediate_full // world
    sl = slice(rank * f, (rank + 1) * f)
    p = {}
    p["router_weight"] = (torch.randn(experts + n_shared, hidden, generator=gen, device=device) * std).to(BF16)
    bias = torch.randn(experts, generator=gen, device=device) * bias_std
    p["router_bias"] = bias.float()
    p["global_scale"] = torch.ones(1, dtype=BF16, device=device)
    gate = (torch.randn(n_shared, intermediate_full, hidden, generator=gen, device=device) * std).to(BF16)
    up = (torch.randn(n_shared, intermediate_full, hidden, generator=gen, device=device) * std).to(BF16)
    down = (torch.randn(n_shared, hidden, intermediate_full, generator=gen, device=device) * std).to(BF16)
    p["shared_gate"] = gate[:, sl].contiguous()
    p["shared_up"] = up[:, sl].contiguous()
    p["shared_down"] = down[:, :, sl].contiguous()
    return p
