"""GPU parity of the grouped tensor-core path (ink_expert_gemm / ink_expert_reduce)
against the CPU oracle and against the per-route GEMV path."""
import numpy as np
import pytest
import torch

import cases
from helpers import BF16, banks_to_device, layer_on_device, max_rel, pointer_table, rel_floor
from oracle import moe as oracle_moe

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.fixture(scope="module")
def ib():
    import inkling_b200

    return inkling_b200


@pytest.fixture(scope="module")
def device():
    return torch.device("cuda", 0)


def _skewed_routing(gen, tokens, experts, k):
    probs = 1.0 / torch.arange(1, experts + 1).float() ** 1.1       # Zipf(s = 1.1)
    perm = torch.randperm(experts, generator=gen)
    return torch.stack([perm[torch.multinomial(probs, k, replacement=False, generator=gen)] for _ in range(tokens)])


@pytest.mark.parametrize("name,tokens", [("mid", 40), ("tp8_slice", 24), ("mid", 200)])
def test_grouped_projections_against_oracle(ib, device, name, tokens):
    c = dict(cases.LAYER_CASES[name], tokens=tokens)
    p, banks, x = cases.make_layer(**c)
    gen = torch.Generator().manual_seed(tokens)
    idx = _skewed_routing(gen, tokens, c["experts"], c["top_k"])
    w = torch.rand(tokens, c["top_k"], generator=gen).to(BF16)
    dev_banks = banks_to_device(banks, device)
    E, d, f, k = c["experts"], c["d"], c["f"], c["top_k"]
    routes = idx.numel()
    capacity = 1 << (routes - 1).bit_length()
    sources = pointer_table(dev_banks, device).view(E, 6)
    i32 = dict(dtype=torch.int32, device=device)
    pointers = torch.zeros(E * 6, dtype=torch.int64, device=device)
    experts, counts = torch.empty(E, **i32), torch.empty(E, **i32)
    rows = torch.full((E, capacity), -1, **i32)
    idx_d, w_d, x_d = idx.to(device), w.to(device), x.to(device)
    ib.kernels.expert_plan[(1,)](idx_d, sources, None, None, None, None, None, torch.empty(0, **i32), pointers,
                                 experts, counts, rows, 0, E, 0, 6, routes, capacity)
    activated = torch.zeros(capacity, f, dtype=BF16, device=device)
    down = torch.zeros(capacity, d, dtype=BF16, device=device)
    groups = min(routes, E)
    ib.kernels.expert_gemm[(1, 1, groups)](x_d, pointers, experts, rows, counts, activated, capacity, 2 * f, d, k,
                                           0, True, 6, 16, 64, 64)
    ib.kernels.expert_gemm[(1, 1, groups)](activated, pointers, experts, rows, counts, down, capacity, d, f, k,
                                           1, True, 6, 16, 64, 64)
    out = torch.zeros(tokens, d, dtype=torch.float32, device=device)
    ib.kernels.expert_reduce[(tokens, 1)](down, idx_d, w_d, pointers, out, d, k, 6, E - 1, 256)
    torch.cuda.synchronize()
    plan = oracle_moe.expert_plan(idx, sources.cpu(), 0, E, 6, capacity)
    want_act = oracle_moe.expert_gemm_reference(x, plan, banks, 0, k, 2 * f, capacity)
    assert max_rel(activated.cpu().float(), want_act.float()) <= 1.6e-2        # BF16 weights there, exact weights here
    want_down = oracle_moe.expert_gemm_reference(activated.cpu(), plan, banks, 1, k, d, capacity)
    assert max_rel(down.cpu().float(), want_down.float()) <= 1.6e-2
    active = torch.ones_like(idx, dtype=torch.bool)
    want_out = oracle_moe.expert_reduce_reference(down.cpu(), idx, w, active, torch.zeros(tokens, d))
    assert max_rel(out.cpu(), want_out) <= 1e-6
    assert max_rel(out.cpu(), oracle_moe.routed_experts_fp32(x, idx, w, banks)) <= TOL


def test_module_switches_to_grouped_path_and_agrees_with_gemv(ib, device):
    """More than 8 tokens go through the grouped GEMMs; the same tokens eight at a time go
    through the per-route GEMV. Both must agree with the float64 oracle."""
    c = dict(cases.LAYER_CASES["mid"], tokens=33)
    p, banks, x = cases.make_layer(**c)
    dp = layer_on_device(p, device)
    experts = ib.ResidentExperts(p["d"], p["f"], None, banks_to_device(banks, device))
    layer = ib.FusedMoE(dp["router_weight"], dp["router_bias"], dp["global_scale"], p["route_scale"], p["top_k"],
                        dp["shared_gate"], dp["shared_up"], dp["shared_down"], experts, None)
    many = layer(x.to(device).unsqueeze(0))[0].float().cpu()
    torch.cuda.synchronize()
    idx, w, gam = layer.topk_indices[:33].cpu(), layer.topk_weights[:33].cpu(), layer.gammas[:33].cpu()
    want = oracle_moe.moe_layer_fp32(x, p, banks, idx, w, gam)
    assert max_rel(many, want) <= TOL
    few = torch.cat([layer(x[i:i + 8].to(device).unsqueeze(0))[0].float().cpu() for i in range(0, 33, 8)])
    assert max_rel(few, want) <= TOL
    assert max_rel(many, few) <= TOL
    layer.experts.check_status()


def test_batched_decode_64_tokens_zipf_at_full_shapes(ib, device):
    """config[3]: 64 tokens through one block of the full shapes, routing skewed by
    Zipf(1.1); grouped path against the per-route GEMV on the same routing."""
    d, f, E, k = 4096, 2048, 256, 6
    banks = ib.make_expert_banks(E, d, f, device, seed=2)
    experts = ib.ResidentExperts(d, f, None, banks.weights)
    gen = torch.Generator().manual_seed(64)
    x = torch.randn(64, d, generator=gen).to(BF16).to(device)
    idx = _skewed_routing(gen, 64, E, k).to(device)
    w = torch.rand(64, k, generator=gen).to(BF16).to(device)
    grouped = experts(x, idx, w).float()
    torch.cuda.synchronize()
    gemv = torch.cat([experts(x[i:i + 8], idx[i:i + 8].contiguous(), w[i:i + 8].contiguous()).float()
                      for i in range(0, 64, 8)])
    torch.cuda.synchronize()
    assert torch.isfinite(grouped).all()
    assert max_rel(grouped, gemv) <= TOL
    experts.check_status()
    # and against the float64 oracle on a few tokens (their experts' banks copied to the host)
    for token in (0, 41):
        ids = idx[token].cpu()
        cpu_banks = {int(e): {n: t.cpu() for n, t in banks.weights[int(e)].items()} for e in ids.tolist()}
        want = oracle_moe.routed_experts_fp32(x[token:token + 1].cpu(), ids.view(1, -1), w[token:token + 1].cpu(), cpu_banks)
        for got in (grouped[token:token + 1], gemv[token:token + 1]):
            assert max_rel(got, want) <= TOL
            assert rel_floor(got, want) <= 0.2
        del cpu_banks


def test_a_prompt_of_2048_tokens_at_full_shapes(ib, device):
    """12 288 routes through one block of the full shapes (a prefill-sized batch: the planner's large path, the
    grouped block-scaled kernel with up to hundreds of routes per expert): sampled tokens against the float64
    oracle, and the whole batch against itself in two halves (the result of a token does not depend on its batch)."""
    d, f, E, k, tokens = 4096, 2048, 256, 6, 2048
    banks = ib.make_expert_banks(E, d, f, device, seed=2)
    experts = ib.ResidentExperts(d, f, None, banks.weights)
    gen = torch.Generator().manual_seed(2048)
    x = torch.randn(tokens, d, generator=gen).to(BF16).to(device)
    idx = _skewed_routing(gen, tokens, E, k).to(device)
    w = torch.rand(tokens, k, generator=gen).to(BF16).to(device)
    whole = experts(x, idx, w).float().clone()
    torch.cuda.synchronize()
    experts.check_status()
    assert torch.isfinite(whole).all()
    halves = torch.cat([experts(x[a:a + 1024], idx[a:a + 1024].contiguous(), w[a:a + 1024].contiguous()).float().clone()
                        for a in (0, 1024)])
    torch.cuda.synchronize()
    assert max_rel(whole, halves) <= 1e-2
    for token in (0, 1023, 2047):
        ids = idx[token].cpu()
        cpu_banks = {int(e): {n: t.cpu() for n, t in banks.weights[int(e)].items()} for e in ids.tolist()}
        want = oracle_moe.routed_experts_fp32(x[token:token + 1].cpu(), ids.view(1, -1), w[token:token + 1].cpu(), cpu_banks)
        assert max_rel(whole[token:token + 1], want) <= TOL
        del cpu_banks


@pytest.mark.parametrize("d,f,E,tokens", [(1024, 512, 32, 40), (2048, 256, 16, 24), (1024, 512, 32, 200)])
def test_block_scaled_projections_against_oracle(ib, device, d, f, E, tokens):
    """ink_expert_gemm_tc: the packed banks straight into tcgen05.mma.kind::mxf4nvf4.block_scale (banks of one
    kind in one allocation, addressed through TMA descriptors), tokens as E2M1 digit rows; experts with more than
    eight routes take several passes. Against the CPU oracle, and against the kernel that expands to FP16."""
    k = 6
    banks = ib.make_expert_banks(E, d, f, device, seed=17)
    experts_module = ib.ResidentExperts(d, f, None, banks.weights)
    assert experts_module.bank_maps is not None
    gen = torch.Generator().manual_seed(tokens)
    x = torch.randn(tokens, d, generator=gen).to(BF16)
    idx = _skewed_routing(gen, tokens, E, k)
    w = torch.rand(tokens, k, generator=gen).to(BF16)
    routes = idx.numel()
    capacity = 1 << (routes - 1).bit_length()
    i32 = dict(dtype=torch.int32, device=device)
    sources = experts_module.sources
    pointers = torch.zeros(E * 6, dtype=torch.int64, device=device)
    experts, counts = torch.empty(E, **i32), torch.empty(E, **i32)
    rows = torch.full((E, capacity), -1, **i32)
    idx_d, w_d, x_d = idx.to(device), w.to(device), x.to(device)
    ib.kernels.expert_plan[(1,)](idx_d, sources, None, None, None, None, None, torch.empty(0, **i32), pointers,
                                 experts, counts, rows, 0, E, 0, 6, routes, capacity)
    groups = min(routes, E)
    status = torch.zeros(1, **i32)
    outs = {}
    for name, maps in (("block_scaled", experts_module.bank_maps), ("fp16", None)):
        activated = torch.zeros(capacity, f, dtype=BF16, device=device)
        down = torch.zeros(capacity, d, dtype=BF16, device=device)
        ib.kernels.expert_gemm[(1, 1, groups)](x_d, pointers, experts, rows, counts, activated, capacity, 2 * f, d, k,
                                               0, True, 6, 16, 64, 64, status=status, bank_maps=maps)
        ib.kernels.expert_gemm[(1, 1, groups)](activated, pointers, experts, rows, counts, down, capacity, d, f, k,
                                               1, True, 6, 16, 64, 64, status=status, bank_maps=maps)
        out = torch.zeros(tokens, d, dtype=torch.float32, device=device)
        ib.kernels.expert_reduce[(tokens, 1)](down, idx_d, w_d, pointers, out, d, k, 6, E - 1, 256)
        torch.cuda.synchronize()
        outs[name] = (activated.cpu(), down.cpu(), out.cpu())
    assert int(status.item()) == 0
    cpu_banks = {e: {n: t.cpu() for n, t in banks.weights[e].items()} for e in range(E)}
    plan = oracle_moe.expert_plan(idx, sources.cpu(), 0, E, 6, capacity)
    activated, down, out = outs["block_scaled"]
    want_act = oracle_moe.expert_gemm_reference(x, plan, cpu_banks, 0, k, 2 * f, capacity)
    assert max_rel(activated.float(), want_act.float()) <= 1.6e-2
    want_down = oracle_moe.expert_gemm_reference(activated, plan, cpu_banks, 1, k, d, capacity)
    assert max_rel(down.float(), want_down.float()) <= 1.6e-2
    assert max_rel(out, oracle_moe.routed_experts_fp32(x, idx, w, cpu_banks)) <= TOL
    assert max_rel(out, outs["fp16"][2]) <= TOL
