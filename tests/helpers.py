"""Shared helpers for the GPU parity tests."""
from __future__ import annotations

import torch

import cases
from oracle import moe as oracle_moe

BF16 = torch.bfloat16


def max_rel(actual, expected) -> float:
    """max_i |a_i - e_i| / max_i |e_i| : the tolerance definition used for layer outputs."""
    actual, expected = torch.as_tensor(actual).double().cpu(), torch.as_tensor(expected).double().cpu()
    return float((actual - expected).abs().max() / expected.abs().max().clamp_min(1e-30))


def rel_floor(actual, expected, floor_fraction: float = 0.05) -> float:
    """max_i |a_i - e_i| / max(|e_i|, floor): the per-element relative error with an absolute
    floor of `floor_fraction` of the largest expected magnitude (elements near zero are
    measured against the floor instead of against themselves)."""
    actual, expected = torch.as_tensor(actual).double().cpu(), torch.as_tensor(expected).double().cpu()
    floor = floor_fraction * expected.abs().max().clamp_min(1e-30)
    return float(((actual - expected).abs() / expected.abs().clamp_min(floor)).max())


def bf16_ulps(actual, expected) -> torch.Tensor:
    """Distance in BF16 units in the last place between two BF16 tensors."""
    a = actual.cpu().to(BF16).view(torch.int16).to(torch.int32)
    e = expected.cpu().to(BF16).view(torch.int16).to(torch.int32)
    # map sign-magnitude to a monotone integer line
    a = torch.where(a < 0, -(a & 0x7FFF), a)
    e = torch.where(e < 0, -(e & 0x7FFF), e)
    return (a - e).abs()


def banks_to_device(banks: dict, device) -> dict:
    """Per-expert bank dictionaries on the device, scale2 as 1-element FP32 tensors."""
    out = {}
    for e, b in banks.items():
        out[e] = {n: (t.reshape(1).float() if n.endswith("scale2") else t).to(device).contiguous()
                  for n, t in b.items()}
    return out


def pointer_table(dev_banks: dict, device, inactive=()) -> torch.Tensor:
    """Flat int64 [(max_expert + 1) * 6] table; experts in `inactive` get a zero row."""
    n = max(dev_banks) + 1
    table = torch.zeros(n, 6, dtype=torch.int64)
    for e, b in dev_banks.items():
        if e not in inactive:
            table[e] = torch.tensor([b[name].data_ptr() for name in cases.BANK_NAMES])
    return table.reshape(-1).to(device)


def layer_on_device(p: dict, device) -> dict:
    return {k: (v.to(device).contiguous() if isinstance(v, torch.Tensor) else v) for k, v in p.items()}


def run_router(ib, p, x, device, with_logits=True):
    t = x.shape[0]
    k, ns = p["top_k"], p["n_shared"]
    w = torch.empty(t, k, dtype=BF16, device=device)
    idx = torch.full((t, k), -1, dtype=torch.int64, device=device)
    gam = torch.empty(t, ns, dtype=BF16, device=device)
    logits = torch.empty(t, p["experts"], dtype=BF16, device=device) if with_logits else None
    ws = ib.kernels.router_workspace(t, p["experts"] + ns, device)
    ib.kernels.router_forward(x.to(device), p["router_weight"].to(device), p["router_bias"].to(device),
                              p["global_scale"].to(device), p["route_scale"], k, ns, w, idx, gam, ws,
                              routed_logits=logits)
    return logits, w, idx, gam, ws


def assert_router_matches(p, x, got_idx, got_w, got_gam, max_ulps=2):
    """Index sets bit-exact against the oracle except on tokens whose top-k set exact
    arithmetic does not determine; weights within `max_ulps` BF16 ulps where the sets agree."""
    _, want_w, want_idx, want_gam = oracle_moe.router(x, p["router_weight"], p["router_bias"], p["global_scale"],
                                                      p["route_scale"], p["top_k"], p["n_shared"])
    fragile = oracle_moe.router_fragile_tokens(x, p["router_weight"], p["router_bias"], p["n_shared"], p["top_k"])
    got_sorted, got_order = got_idx.cpu().sort(-1)
    want_sorted, want_order = want_idx.sort(-1)
    same = (got_sorted == want_sorted).all(-1)
    assert bool((same | fragile).all()), f"top-k sets differ on non-fragile tokens: {(~(same | fragile)).nonzero().flatten().tolist()}"
    # every chosen expert must at least tie the k-th score of the oracle's choice
    scores = oracle_moe.router_choice_scores(x, p["router_weight"], p["router_bias"], p["n_shared"])
    kth = scores.gather(-1, want_idx).min(-1).values
    if not bool(fragile.any()):
        assert bool((scores.gather(-1, got_idx.cpu()) >= kth[:, None]).all())
    rows = same.nonzero().flatten()
    ulps_w = bf16_ulps(got_w.cpu().gather(-1, got_order)[rows], want_w.gather(-1, want_order)[rows])
    ulps_g = bf16_ulps(got_gam.cpu()[rows], want_gam[rows])
    assert int(ulps_w.max()) <= max_ulps and int(ulps_g.max()) <= max_ulps, (int(ulps_w.max()), int(ulps_g.max()))
    return same, fragile
