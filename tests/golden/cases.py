"""Seeded input builders shared by the fixture generator (make_golden.py) and the
tests. Inputs are rebuilt from a seed on whichever machine runs the test (same torch
build on both); a checksum of every rebuilt input is stored with the fixture so that a
drift in the generator is reported as such and not as a parity failure."""
from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from oracle import nvfp4  # noqa: E402

BF16 = torch.bfloat16
BANK_NAMES = ("gate_up_proj", "gate_up_proj_scale", "gate_up_proj_scale2",
              "down_proj", "down_proj_scale", "down_proj_scale2")

# name -> dict(d, f, experts, n_shared, top_k, tokens, seed, bias)
LAYER_CASES = {
    # smallest widths the reference GEMV accepts (width % 32 == 0 and 128 % (width/32) == 0)
    "tiny": dict(d=128, f=64, experts=8, n_shared=2, top_k=2, tokens=5, seed=1, bias="linspace"),
    "small": dict(d=256, f=128, experts=16, n_shared=2, top_k=6, tokens=3, seed=2, bias="zero"),
    "mid": dict(d=1024, f=512, experts=32, n_shared=2, top_k=6, tokens=2, seed=3, bias="randn"),
    "tp8_slice": dict(d=2048, f=256, experts=16, n_shared=2, top_k=6, tokens=1, seed=4, bias="randn"),
}


def checksum(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        if isinstance(t, torch.Tensor):
            t = t.detach().cpu().contiguous().reshape(-1)
            t = t.view(torch.uint8) if t.dtype != torch.bool else t.to(torch.uint8)
            h.update(t.numpy().tobytes())
        else:
            h.update(np.asarray(t).tobytes())
    return h.hexdigest()[:16]


def make_expert_banks(gen, experts: int, d: int, f: int, std: float = 0.02) -> dict:
    """NVFP4 banks per expert in the checkpoint layout: gate_up rows interleaved
    (even = gate, odd = up), codes two per byte, one E4M3 scale per 16 columns."""
    banks = {}
    for e in range(experts):
        gate_up = torch.randn(2 * f, d, generator=gen) * std
        down = torch.randn(d, f, generator=gen) * std
        c0, s0, g0 = nvfp4.quantize_nvfp4(gate_up)
        c1, s1, g1 = nvfp4.quantize_nvfp4(down)
        banks[e] = dict(zip(BANK_NAMES, (c0, s0, g0, c1, s1, g1)))
    return banks


def make_layer(d, f, experts, n_shared, top_k, tokens, seed, bias, std=0.02, route_scale=8.0,
               global_scale=1.0):
    gen = torch.Generator().manual_seed(seed)
    p = dict(d=d, f=f, experts=experts, n_shared=n_shared, top_k=top_k, route_scale=route_scale)
    p["router_weight"] = (torch.randn(experts + n_shared, d, generator=gen) * std).to(BF16)
    if bias == "zero":
        p["router_bias"] = torch.zeros(experts)
    elif bias == "linspace":
        p["router_bias"] = torch.linspace(-0.3, 0.3, experts)
    else:
        p["router_bias"] = torch.randn(experts, generator=gen) * 0.05
    p["global_scale"] = torch.full((1,), global_scale).to(BF16)
    p["shared_gate"] = (torch.randn(n_shared, f, d, generator=gen) * std).to(BF16)
    p["shared_up"] = (torch.randn(n_shared, f, d, generator=gen) * std).to(BF16)
    p["shared_down"] = (torch.randn(n_shared, d, f, generator=gen) * std).to(BF16)
    banks = make_expert_banks(gen, experts, d, f, std)
    x = torch.randn(tokens, d, generator=gen).to(BF16)
    return p, banks, x


def layer_checksum(p, banks, x) -> str:
    parts = [x, p["router_weight"], p["router_bias"], p["shared_gate"], p["shared_up"], p["shared_down"]]
    for e in sorted(banks):
        parts += [banks[e][n] for n in BANK_NAMES]
    return checksum(*parts)


def dispatch_fixture():
    """Index/weight pattern of the reference's expert test (tests/test_model_parity.py:
    230-233): repeated experts, unequal weights, a zero weight and an unused expert."""
    indices = torch.tensor([[0, 1], [1, 2], [2, 0], [0, 2], [1, 0]])
    weights = torch.tensor([[0.2, 0.8], [0.7, 0.3], [0.4, 0.6], [0.0, 1.0], [0.6, 0.4]])
    return indices, weights


# ------------------------------------------------------------------- glue cases
EPS = 1e-6
GLUE_SEED = 77


def glue_inputs(gen):
    """RMS norm: x BF16 [3, 256] with rows of very different scale, weight BF16 [256]."""
    x = (torch.randn(3, 256, generator=gen) * torch.tensor([[0.05], [1.0], [30.0]])).to(BF16)
    w = (1.0 + 0.2 * torch.randn(256, generator=gen)).to(BF16)
    return x, w


def sconv_inputs(gen, bs: int = 2, d: int = 256, k: int = 4):
    """Short convolution: K consecutive tokens BF16 [bs, K, d] (the last is the decode
    token, the others its history), taps FP32 [d, K] (the checkpoint keeps the convolutions in
    FP32, my_inkling/model.py:743-747), decoder residual BF16 [bs, K, d]."""
    seq = torch.randn(bs, k, d, generator=gen).to(BF16)
    taps = torch.randn(d, k, generator=gen) * 0.3
    residual = torch.randn(bs, k, d, generator=gen).to(BF16)
    return seq, taps, residual


def stack_cases() -> list[dict]:
    """Three blocks of the 'small' shape with their own seeds (first block's x is the input)."""
    return [dict(LAYER_CASES["small"], tokens=1, seed=40 + i, bias="randn") for i in range(3)]


def stack_norm_weight(d: int) -> torch.Tensor:
    gen = torch.Generator().manual_seed(GLUE_SEED + 1)
    return (1.0 + 0.1 * torch.randn(d, generator=gen)).to(BF16)


def bf16_banks(banks: dict) -> dict:
    """BF16 expert banks (pointer stride 2: gate_up_proj, down_proj) with the values of the
    NVFP4 banks: what an unquantised layer of the same experts would hold."""
    return {e: dict(gate_up_proj=nvfp4.dequant_bf16(b["gate_up_proj"], b["gate_up_proj_scale"], b["gate_up_proj_scale2"]).contiguous(),
                    down_proj=nvfp4.dequant_bf16(b["down_proj"], b["down_proj_scale"], b["down_proj_scale2"]).contiguous())
            for e, b in banks.items()}
