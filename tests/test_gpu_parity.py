"""GPU parity: the CUDA path (through the C ABI) against the CPU oracle and against the
fixtures produced by the reference's own code. Tolerance for layer outputs:
max|y - ref| / max|ref| <= 2e-2 against the FP32-accumulated oracle; router top-k sets
and the expert plan bit-exact."""
import numpy as np
import pytest
import torch

import cases
from helpers import (BF16, assert_router_matches, banks_to_device, bf16_ulps, layer_on_device, max_rel,
                     pointer_table, run_router)
from oracle import moe as oracle_moe

pytestmark = pytest.mark.gpu
TOL = 2e-2
NAMES = list(cases.LAYER_CASES)


@pytest.fixture(scope="module")
def ib():
    import inkling_b200

    return inkling_b200


@pytest.fixture(scope="module")
def device():
    assert torch.cuda.is_available()
    return torch.device("cuda", 0)


@pytest.fixture(scope="module", params=NAMES)
def case(request):
    name = request.param
    p, banks, x = cases.make_layer(**cases.LAYER_CASES[name])
    return name, p, banks, x


def g(golden, key, dtype=None):
    t = torch.from_numpy(golden[key])
    return t.to(dtype) if dtype is not None else t


# ------------------------------------------------------------------ router
def test_router_against_oracle_and_reference_class(ib, device, case, golden):
    name, p, banks, x = case
    logits, w, idx, gam, _ = run_router(ib, p, x, device)
    torch.cuda.synchronize()
    same, fragile = assert_router_matches(p, x, idx, w, gam)
    # fixtures written by the reference's MyInklingTopkRouter
    want_idx = g(golden, f"{name}/router_indices")
    rows = (~fragile).nonzero().flatten()
    assert torch.equal(idx.cpu().sort(-1).values[rows], want_idx.sort(-1).values[rows])
    assert int(bf16_ulps(logits.cpu(), g(golden, f"{name}/router_logits", BF16)).max()) <= 1


def test_router_baseline_shape_ties_and_bias(ib, device):
    """256 routed + 2 shared experts, hidden 4096, top-6: zero bias (frequent BF16 score
    ties) and a seeded FP32 bias."""
    for bias in ("zero", "randn"):
        gen = torch.Generator().manual_seed(11)
        p = dict(experts=256, n_shared=2, top_k=6, route_scale=8.0)
        p["router_weight"] = (torch.randn(258, 4096, generator=gen) * 0.02).to(BF16)
        p["router_bias"] = torch.zeros(256) if bias == "zero" else torch.randn(256, generator=gen) * 0.05
        p["global_scale"] = torch.full((1,), 1.3).to(BF16)
        x = torch.randn(48, 4096, generator=gen).to(BF16)
        for chunk in (x[:1], x[1:8], x[8:48]):
            _, w, idx, gam, _ = run_router(ib, p, chunk, device, with_logits=False)
            same, fragile = assert_router_matches(p, chunk, idx, w, gam)
            assert idx.min() >= 0 and idx.max() < 256
            assert (idx.cpu().sort(-1).values.diff(dim=-1) > 0).all(), "an expert was chosen twice"


def test_router_workspace_is_reusable(ib, device):
    p, banks, x = cases.make_layer(**cases.LAYER_CASES["small"])
    t, k, ns = x.shape[0], p["top_k"], p["n_shared"]
    ws = ib.kernels.router_workspace(t, p["experts"] + ns, device)
    outs = []
    for _ in range(3):
        w = torch.empty(t, k, dtype=BF16, device=device)
        idx = torch.empty(t, k, dtype=torch.int64, device=device)
        gam = torch.empty(t, ns, dtype=BF16, device=device)
        ib.kernels.router_forward(x.to(device), p["router_weight"].to(device), p["router_bias"].to(device),
                                  p["global_scale"].to(device), p["route_scale"], k, ns, w, idx, gam, ws)
        outs.append((w.clone(), idx.clone(), gam.clone()))
    torch.cuda.synchronize()
    for w, idx, gam in outs[1:]:
        assert torch.equal(w, outs[0][0]) and torch.equal(idx, outs[0][1]) and torch.equal(gam, outs[0][2])


# -------------------------------------------------------------------- plan
def _run_plan(ib, device, indices, E, capacity, start=0, local=None, max_expert=None, sources=None):
    local = E if local is None else local
    max_expert = start + local - 1 if max_expert is None else max_expert
    if sources is None:
        sources = (torch.arange(local * 6, dtype=torch.int64).reshape(local, 6) + 1) * 256
    i32 = dict(dtype=torch.int32, device=device)
    pointers = torch.full(((max_expert + 1) * 6,), 0, dtype=torch.int64, device=device)
    experts, counts = torch.full((local,), -9, **i32), torch.full((local,), -9, **i32)
    rows = torch.full((local, capacity), -1, **i32)
    routes = indices.numel()
    ib.kernels.expert_plan[(1,)](indices.to(device), sources.to(device), None, None, None, None, None,
                                 torch.empty(0, **i32), pointers, experts, counts, rows, start, local, 0, 6,
                                 routes, capacity)
    torch.cuda.synchronize()
    return dict(experts=experts.cpu().numpy(), counts=counts.cpu().numpy(), rows=rows.cpu().numpy(),
                pointers=pointers.cpu().numpy()), sources


@pytest.mark.parametrize("n", range(5))
def test_plan_matches_reference_triton_fixture(ib, device, golden, n):
    idx = torch.from_numpy(golden[f"plan{n}/indices"])
    E = golden[f"plan{n}/experts"].shape[0]
    capacity = golden[f"plan{n}/rows"].shape[1]
    got, _ = _run_plan(ib, device, idx, E, capacity)
    for key in ("experts", "counts", "rows", "pointers"):
        assert np.array_equal(got[key], golden[f"plan{n}/{key}"]), key


@pytest.mark.parametrize("tokens,E,k,start,local", [(1, 256, 6, 0, 256), (8, 256, 6, 0, 256), (64, 256, 6, 0, 256),
                                                     (300, 256, 6, 0, 256), (2048, 256, 6, 0, 256),
                                                     (40, 64, 4, 16, 32), (700, 2048, 2, 0, 2048)])
def test_plan_against_oracle(ib, device, tokens, E, k, start, local):
    gen = torch.Generator().manual_seed(tokens * 7 + E)
    # skewed routing: a few hot experts, many empty ones, ids outside the local range
    probs = 1.0 / torch.arange(1, E + 1).float() ** 1.1
    idx = torch.stack([torch.multinomial(probs, k, replacement=False, generator=gen) for _ in range(tokens)])
    routes = idx.numel()
    capacity = 1 << (routes - 1).bit_length()
    got, sources = _run_plan(ib, device, idx, E, capacity, start=start, local=local, max_expert=E - 1)
    want = oracle_moe.expert_plan(idx, sources, start, local, 6, capacity, max_expert=E - 1)
    for key in ("experts", "counts", "rows", "pointers"):
        assert np.array_equal(got[key], want[key]), key


def test_router_and_plan_in_one_launch(ib, device):
    p, banks, x = cases.make_layer(**cases.LAYER_CASES["small"])
    t, k, ns, E = x.shape[0], p["top_k"], p["n_shared"], p["experts"]
    i32 = dict(dtype=torch.int32, device=device)
    w = torch.empty(t, k, dtype=BF16, device=device)
    idx = torch.empty(t, k, dtype=torch.int64, device=device)
    gam = torch.empty(t, ns, dtype=BF16, device=device)
    ws = ib.kernels.router_workspace(t, E + ns, device)
    sources = ((torch.arange(E * 6, dtype=torch.int64).reshape(E, 6) + 1) * 256).to(device)
    capacity = 32
    pointers = torch.zeros(E * 6, dtype=torch.int64, device=device)
    experts, counts = torch.empty(E, **i32), torch.empty(E, **i32)
    rows = torch.full((E, capacity), -1, **i32)
    ib.kernels.router_plan_forward(x.to(device), p["router_weight"].to(device), p["router_bias"].to(device),
                                   p["global_scale"].to(device), p["route_scale"], k, ns, w, idx, gam, ws,
                                   sources, pointers, experts, counts, rows, 0, E, 6, capacity)
    torch.cuda.synchronize()
    assert_router_matches(p, x, idx, w, gam)
    want = oracle_moe.expert_plan(idx.cpu(), sources.cpu(), 0, E, 6, capacity)
    assert np.array_equal(experts.cpu().numpy(), want["experts"])
    assert np.array_equal(counts.cpu().numpy(), want["counts"])
    assert np.array_equal(rows.cpu().numpy(), want["rows"])
    assert np.array_equal(pointers.cpu().numpy(), want["pointers"])


# ------------------------------------------------------------ routed GEMV
def _routed(ib, device, x, idx, w, dev_banks, inactive=(), max_expert=None, status=None):
    t, d = x.shape
    f = next(iter(dev_banks.values()))["gate_up_proj"].shape[0] // 2
    pointers = pointer_table(dev_banks, device, inactive)
    activated = torch.zeros(max(t * idx.shape[1], 1), f, dtype=BF16, device=device)
    out = torch.full((t, d), float("nan"), dtype=torch.float32, device=device)
    ib.kernels.routed_decode(x.to(device), idx.to(device), w.to(device), pointers, activated, out,
                             max(dev_banks) if max_expert is None else max_expert, True, status=status)
    torch.cuda.synchronize()
    return activated.cpu(), out.cpu()


def test_gemv_against_oracle_and_reference_cuda_file(ib, device, case, golden):
    name, p, banks, x = case
    idx = g(golden, f"{name}/routing_indices")
    w = g(golden, f"{name}/routing_weights", BF16)
    dev_banks = banks_to_device(banks, device)
    act, out = _routed(ib, device, x, idx, w, dev_banks)
    assert not torch.isnan(out).any()
    want_act, want_out = oracle_moe.routed_decode_reference(x, idx, w, banks)
    assert max_rel(act.float(), want_act.float()) <= 8e-3      # one BF16 ulp of the largest activation
    assert max_rel(out, want_out) <= 1e-2
    assert max_rel(out, oracle_moe.routed_experts_fp32(x, idx, w, banks)) <= TOL
    # the reference's own kernels/routed_decode.cu, run on the CPU
    assert max_rel(act.float(), g(golden, f"{name}/gemv_activated")) <= 8e-3
    assert max_rel(out, g(golden, f"{name}/gemv_out")) <= 1e-2


def test_gemv_skips_inactive_and_flags_bad_ids(ib, device):
    p, banks, x = cases.make_layer(**cases.LAYER_CASES["small"])
    dev_banks = banks_to_device(banks, device)
    idx = torch.tensor([[0, 3, 5, 7, 9, 11], [3, 3, 0, 1, 2, 15], [15, 14, 13, 12, 11, 10]])
    w = torch.rand(3, 6).to(BF16)
    w[1, 2] = 0
    inactive = (3, 12)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    act, out = _routed(ib, device, x, idx, w, dev_banks, inactive=inactive, status=status)
    assert int(status.item()) == 0
    kept = {e: b for e, b in banks.items() if e not in inactive}
    assert max_rel(out, oracle_moe.routed_experts_fp32(x, idx, w, kept)) <= TOL
    # an id outside [0, max_expert] is skipped (as in the reference) and reported
    bad = idx.clone()
    bad[0, 0], bad[2, 5] = 16, -1
    act, out_bad = _routed(ib, device, x, bad, w, dev_banks, status=status)
    assert int(status.item()) & 1
    assert max_rel(out_bad, oracle_moe.routed_experts_fp32(x, bad, w, banks)) <= TOL


def test_gemv_empty_batch(ib, device):
    p, banks, x = cases.make_layer(**cases.LAYER_CASES["small"])
    dev_banks = banks_to_device(banks, device)
    idx = torch.zeros(0, 6, dtype=torch.int64)
    act, out = _routed(ib, device, x[:0], idx, torch.zeros(0, 6).to(BF16), dev_banks)
    assert out.shape == (0, x.shape[1])


def test_gemv_rejects_bad_arguments(ib, device):
    p, banks, x = cases.make_layer(**cases.LAYER_CASES["small"])
    dev_banks = banks_to_device(banks, device)
    idx = torch.zeros(1, 6, dtype=torch.int64)
    w = torch.ones(1, 6).to(BF16)
    with pytest.raises(AssertionError):
        _routed(ib, device, x[:1].float(), idx, w, dev_banks)           # dtype, as the reference asserts
    pointers = pointer_table(dev_banks, device)
    activated = torch.zeros(6, 96, dtype=BF16, device=device)             # 96 is not a supported width
    out = torch.zeros(1, 256, dtype=torch.float32, device=device)
    with pytest.raises(RuntimeError, match="unsupported"):
        ib.kernels.routed_decode(x[:1].to(device), idx.to(device), w.to(device), pointers, activated, out, 15, True)
    with pytest.raises(RuntimeError, match="unsupported"):               # the same for BF16 banks (quantized=False)
        ib.kernels.routed_decode(x[:1].to(device), idx.to(device), w.to(device), pointers, activated, out, 15, False)


# ------------------------------------------------------------- whole layer
def _fused_layer(ib, device, p, banks, x, group=None):
    dp = layer_on_device(p, device)
    dev_banks = banks_to_device(banks, device)
    experts = ib.ResidentExperts(p["d"], p["f"], group, dev_banks)
    layer = ib.FusedMoE(dp["router_weight"], dp["router_bias"], dp["global_scale"], p["route_scale"], p["top_k"],
                        dp["shared_gate"], dp["shared_up"], dp["shared_down"], experts, group)
    return layer


def test_layer_against_oracle_and_reference_class(ib, device, case, golden):
    name, p, banks, x = case
    layer = _fused_layer(ib, device, p, banks, x)
    out = layer(x.to(device).unsqueeze(0))[0]
    torch.cuda.synchronize()
    t = x.shape[0]
    idx, w, gam = layer.topk_indices[:t].cpu(), layer.topk_weights[:t].cpu(), layer.gammas[:t].cpu()
    same, fragile = assert_router_matches(p, x, idx, w, gam)
    # expert arithmetic for the routing the device chose
    assert max_rel(out.float(), oracle_moe.moe_layer_fp32(x, p, banks, idx, w, gam)) <= TOL
    if bool(same.all()):
        assert max_rel(out.float(), g(golden, f"{name}/moe_out")) <= TOL   # the reference's MyInklingMoE
    layer.experts.check_status()


def test_resident_experts_module_is_a_drop_in(ib, device, golden):
    """forward(hidden, top_k_index, top_k_weights) as the reference's experts module,
    on the reference test's dispatch pattern (repeated experts, a zero weight, an unused
    expert)."""
    p, banks, x = cases.make_layer(**cases.LAYER_CASES["tiny"])
    idx, w = cases.dispatch_fixture()
    experts = ib.ResidentExperts(p["d"], p["f"], None, banks_to_device(banks, device))
    out = experts(x.to(device), idx.to(device), w.to(BF16).to(device))
    torch.cuda.synchronize()
    assert out.dtype == BF16 and out.shape == x.shape
    assert max_rel(out.float(), oracle_moe.routed_experts_fp32(x, idx, w.to(BF16), banks)) <= TOL
    assert max_rel(out.float(), g(golden, "tiny/dispatch_out")) <= TOL
    # the plan tables the module keeps are those of the reference's planner
    assert np.array_equal(experts.experts.cpu().numpy(), golden["tiny/plan_experts"])
    assert np.array_equal(experts.counts.cpu().numpy(), golden["tiny/plan_counts"])


def test_more_tokens_than_one_gemv_batch(ib, device):
    c = dict(cases.LAYER_CASES["small"], tokens=19)
    p, banks, x = cases.make_layer(**c)
    layer = _fused_layer(ib, device, p, banks, x)
    out = layer(x.to(device).view(1, 19, -1))[0]
    torch.cuda.synchronize()
    idx, w, gam = layer.topk_indices[:19].cpu(), layer.topk_weights[:19].cpu(), layer.gammas[:19].cpu()
    assert max_rel(out.float(), oracle_moe.moe_layer_fp32(x, p, banks, idx, w, gam)) <= TOL


def test_graph_replay_equals_eager(ib, device):
    p, banks, x = cases.make_layer(**cases.LAYER_CASES["mid"])
    layer = _fused_layer(ib, device, p, banks, x)
    xs = x.to(device).unsqueeze(0)
    eager = layer(xs).clone()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(3):
            layer(xs)
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    static_in = xs.clone()
    with torch.cuda.graph(graph, stream=stream):
        static_out = layer(static_in)
    for scale in (1.0, 0.5):
        static_in.copy_(xs * scale)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(static_out, layer(xs * scale))
    assert torch.equal(eager, layer(xs))


def test_tensor_parallel_slices_sum_to_the_whole(ib, device):
    """Two ranks' slices (FFN width cut as the reference shards it) run one after the
    other on one GPU; their FP32 partials summed equal the unsharded layer."""
    p, banks, x = cases.make_layer(**cases.LAYER_CASES["mid"])
    whole = _fused_layer(ib, device, p, banks, x)
    ref = whole(x.to(device).unsqueeze(0))[0].float().cpu()
    total = torch.zeros_like(ref)
    for rank in range(2):
        sp = dict(p, f=p["f"] // 2)
        sp["shared_gate"], sp["shared_up"], sp["shared_down"] = oracle_moe.shard_shared(
            p["shared_gate"], p["shared_up"], p["shared_down"], rank, 2)
        sbanks = {e: oracle_moe.shard_banks(b, rank, 2) for e, b in banks.items()}
        part = _fused_layer(ib, device, sp, sbanks, x)
        part(x.to(device).unsqueeze(0))
        total += part.partial[: x.shape[0]].cpu()
    assert max_rel(total, ref) <= 1e-2
    idx, w, gam = whole.topk_indices[: x.shape[0]].cpu(), whole.topk_weights[: x.shape[0]].cpu(), whole.gammas[: x.shape[0]].cpu()
    assert max_rel(total, oracle_moe.moe_layer_fp32(x, p, banks, idx, w, gam)) <= TOL


# ------------------------------------------------ BASELINE sizes: properties
@pytest.fixture(scope="module")
def baseline_layer(ib, device):
    """config[1]: hidden 4096, 256 NVFP4 experts of width 2048, 2 shared experts, top-6."""
    d, f, E, ns, k = 4096, 2048, 256, 2, 6
    banks = ib.make_expert_banks(E, d, f, device, seed=0)
    lp = ib.make_layer_params(d, f, E, ns, device, seed=0)
    experts = ib.ResidentExperts(d, f, None, banks.weights)
    layer = ib.FusedMoE(lp["router_weight"], lp["router_bias"], lp["global_scale"], 8.0, k, lp["shared_gate"],
                        lp["shared_up"], lp["shared_down"], experts, None)
    return layer, banks, lp


def test_baseline_shape_against_oracle(ib, device, baseline_layer):
    """One decode token at the full shapes; only the experts the router picked are
    brought to the CPU for the float64 oracle."""
    layer, banks, lp = baseline_layer
    gen = torch.Generator().manual_seed(123)
    x = torch.randn(1, 4096, generator=gen).to(BF16)
    out = layer(x.to(device).unsqueeze(0))[0]
    torch.cuda.synchronize()
    idx, w, gam = layer.topk_indices[:1].cpu(), layer.topk_weights[:1].cpu(), layer.gammas[:1].cpu()
    p = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in lp.items()}
    p.update(experts=256, n_shared=2, top_k=6, route_scale=8.0)
    assert_router_matches(p, x, idx, w, gam)
    cpu_banks = {int(e): {n: t.cpu() for n, t in banks.weights[int(e)].items()} for e in idx.flatten()}
    want = oracle_moe.moe_layer_fp32(x, p, cpu_banks, idx, w, gam)
    assert max_rel(out.float(), want) <= TOL
    # the launch-by-launch path (two tokens) leaves the gate/up activations in the module's scratch
    x2 = torch.cat([x, x])
    layer(x2.to(device).unsqueeze(0))
    torch.cuda.synchronize()
    idx2, w2 = layer.topk_indices[:1].cpu(), layer.topk_weights[:1].cpu()
    banks2 = {int(e): {n: t.cpu() for n, t in banks.weights[int(e)].items()} for e in idx2.flatten()}
    act_ref, routed_ref = oracle_moe.routed_decode_reference(x, idx2, w2, banks2)
    assert max_rel(layer.experts.activated[:6].cpu().float(), act_ref.float()) <= 8e-3


def test_baseline_shape_properties(ib, device, baseline_layer):
    """Size-independent properties at the full shapes: (1) the routed sum is the FP32 sum,
    in choice order, of the single-route outputs (each term is already BF16-rounded);
    (2) doubling the router weights doubles the routed output exactly; (3) 8 tokens in
    one call equal 8 calls of one token."""
    layer, banks, lp = baseline_layer
    ex = layer.experts
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(8, 4096, generator=gen).to(BF16).to(device)
    idx = torch.stack([torch.randperm(256, generator=gen)[:6] for _ in range(8)]).to(device)
    w = torch.rand(8, 6, generator=gen).to(BF16).to(device)

    def run(xx, ii, ww, pointers=None):
        out = torch.empty(xx.shape[0], 4096, dtype=torch.float32, device=device)
        act = torch.empty(xx.shape[0] * 6, 2048, dtype=BF16, device=device)
        ib.kernels.routed_decode(xx, ii, ww, ex.pointers if pointers is None else pointers, act, out, 255, True)
        return out

    full_table = ex.sources.reshape(-1).clone()
    base = run(x, idx, w, full_table)
    # (3)
    singles = torch.cat([run(x[i:i + 1], idx[i:i + 1].clone(), w[i:i + 1].clone(), full_table) for i in range(8)])
    assert torch.equal(base, singles)
    # (2)
    assert torch.equal(run(x, idx, (w.float() * 2).to(BF16), full_table), base * 2)
    # (1) token 0: one route at a time (the others point at inactive experts)
    total = torch.zeros(4096, dtype=torch.float32, device=device)
    for choice in range(6):
        table = torch.zeros_like(full_table).view(-1, 6)
        e = int(idx[0, choice])
        table[e] = full_table.view(-1, 6)[e]
        total += run(x[:1], idx[:1].clone(), w[:1].clone(), table.reshape(-1))[0]
    assert torch.equal(total, base[0])
    torch.cuda.synchronize()
