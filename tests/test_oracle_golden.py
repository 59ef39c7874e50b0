"""The CPU oracle against fixtures produced by running the reference itself
(tests/golden/make_golden.py): its PyTorch classes, its Triton kernels under the
interpreter and its CUDA C file compiled for the CPU."""
import numpy as np
import pytest
import torch

import cases
from oracle import moe, nvfp4

BF16 = torch.bfloat16
NAMES = list(cases.LAYER_CASES)


def max_rel(actual, expected):
    actual, expected = torch.as_tensor(actual).double(), torch.as_tensor(expected).double()
    return float((actual - expected).abs().max() / expected.abs().max().clamp_min(1e-30))


@pytest.fixture(scope="module", params=NAMES)
def case(request, golden):
    name = request.param
    p, banks, x = cases.make_layer(**cases.LAYER_CASES[name])
    stored = bytes(golden[f"{name}/checksum"]).decode()
    assert cases.layer_checksum(p, banks, x) == stored, "seeded inputs drifted from the fixture's"
    return name, p, banks, x


def g(golden, key, dtype=None):
    t = torch.from_numpy(golden[key])
    return t.to(dtype) if dtype is not None else t


def test_e4m3_table_matches_torch_float8():
    table = nvfp4.e4m3_table()
    native = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float()
    keep = ~torch.isnan(native)
    assert torch.equal(table[keep], native[keep])
    assert table[0x7F] == 480 and table[0xFF] == -480  # no NaN code in the reference table


def test_quantiser_round_trip_is_idempotent():
    gen = torch.Generator().manual_seed(5)
    w = torch.randn(32, 256, generator=gen) * 0.02
    c, s, s2 = nvfp4.quantize_nvfp4(w)
    deq = nvfp4.dequant_exact(c, s, s2).float()
    assert max_rel(deq, w) < 0.2
    c2, s_2, s22 = nvfp4.quantize_nvfp4(deq)
    assert max_rel(nvfp4.dequant_exact(c2, s_2, s22), deq) < 0.13


def test_router_matches_reference_class(case, golden):
    name, p, banks, x = case
    logits, w, idx, gam = moe.router(x, p["router_weight"], p["router_bias"], p["global_scale"],
                                     p["route_scale"], p["top_k"], p["n_shared"])
    assert torch.equal(logits.float(), g(golden, f"{name}/router_logits"))
    want_idx = g(golden, f"{name}/router_indices")
    # topk(sorted=False) order is unspecified: compare as the reference's own test does
    got_sorted, order = idx.sort(-1)
    want_sorted, want_order = want_idx.sort(-1)
    assert torch.equal(got_sorted, want_sorted)
    assert torch.equal(w.float().gather(-1, order), g(golden, f"{name}/router_weights").gather(-1, want_order))
    assert torch.equal(gam.float(), g(golden, f"{name}/router_gammas"))


def test_shared_experts_match_reference_class(case, golden):
    name, p, banks, x = case
    gam = g(golden, f"{name}/router_gammas", BF16)
    out = moe.shared_experts_reference(x, gam, p["shared_gate"], p["shared_up"], p["shared_down"])
    assert max_rel(out.float(), g(golden, f"{name}/shared_out")) < 1e-2
    fp = moe.shared_experts_fp32(x, gam, p["shared_gate"], p["shared_up"], p["shared_down"])
    assert max_rel(out.float(), fp) < 2e-2


def test_dequant_expert_loop_matches_reference_class(case, golden):
    name, p, banks, x = case
    idx = g(golden, f"{name}/router_indices")
    w = g(golden, f"{name}/router_weights", BF16)
    out = moe.routed_experts_dequant_reference(x, idx, w, banks)
    want = g(golden, f"{name}/experts_out")
    assert max_rel(out.float(), want) < 1e-2
    assert max_rel(want, moe.routed_experts_fp32(x, idx, w, banks)) < 2e-2


def test_dispatch_fixture_of_reference_test(golden):
    p, banks, x = cases.make_layer(**cases.LAYER_CASES["tiny"])
    idx, w = cases.dispatch_fixture()
    out = moe.routed_experts_dequant_reference(x, idx, w.to(BF16), banks)
    assert max_rel(out.float(), g(golden, "tiny/dispatch_out")) < 1e-2


def test_layer_matches_reference_class(case, golden):
    name, p, banks, x = case
    out, idx, w, gam = moe.moe_layer_reference(x, p, banks)
    want = g(golden, f"{name}/moe_out")
    assert max_rel(out.float(), want) < 1e-2
    assert max_rel(want, moe.moe_layer_fp32(x, p, banks, idx, w, gam)) < 2e-2


def _plan_inputs(name, golden, c):
    idx = g(golden, f"{name}/routing_indices")
    routes = idx.numel()
    capacity = 1 << (routes - 1).bit_length()
    sources = np.arange(c["experts"] * 6, dtype=np.int64).reshape(-1, 6) + 1
    return idx, capacity, sources


def test_plan_matches_reference_triton_kernel(case, golden):
    name, p, banks, x = case
    c = cases.LAYER_CASES[name]
    idx, capacity, sources = _plan_inputs(name, golden, c)
    plan = moe.expert_plan(idx, sources, 0, c["experts"], 6, capacity)
    assert np.array_equal(plan["experts"], golden[f"{name}/plan_experts"])
    assert np.array_equal(plan["counts"], golden[f"{name}/plan_counts"])
    assert np.array_equal(plan["rows"], golden[f"{name}/plan_rows"])  # untouched cells hold the -1 prefill
    active = plan["pointers"].reshape(-1, 6)[:, 0] != 0
    assert np.array_equal(active, golden[f"{name}/plan_active"])


@pytest.mark.parametrize("n", range(5))
def test_plan_random_routings(golden, n):
    idx = golden[f"plan{n}/indices"]
    E = golden[f"plan{n}/experts"].shape[0]
    capacity = golden[f"plan{n}/rows"].shape[1]
    sources = (np.arange(E * 6, dtype=np.int64).reshape(E, 6) + 1) * 256
    plan = moe.expert_plan(idx, sources, 0, E, 6, capacity)
    for key in ("experts", "counts", "rows", "pointers"):
        assert np.array_equal(plan[key], golden[f"plan{n}/{key}"]), key


def test_grouped_gemm_and_reduce_match_reference_triton_kernels(case, golden):
    """Pins the NVFP4 decode arithmetic: the reference kernel dequantises inline."""
    name, p, banks, x = case
    c = cases.LAYER_CASES[name]
    idx, capacity, sources = _plan_inputs(name, golden, c)
    # FP32 activations: see make_golden.py (the interpreter cannot do BF16)
    w = g(golden, f"{name}/routing_weights").float()
    plan = moe.expert_plan(idx, sources, 0, c["experts"], 6, capacity)
    act = moe.expert_gemm_reference(x.float(), plan, banks, 0, idx.shape[1], 2 * c["f"], capacity)
    want_act = g(golden, f"{name}/gemm_activated")
    assert max_rel(act, want_act) < 2e-6  # FP32 summation order only
    down = moe.expert_gemm_reference(want_act, plan, banks, 1, idx.shape[1], c["d"], capacity)
    want_down = g(golden, f"{name}/gemm_down")
    assert max_rel(down, want_down) < 2e-6
    active = torch.ones_like(idx, dtype=torch.bool)
    out = moe.expert_reduce_reference(want_down, idx, w, active, torch.zeros(x.shape[0], c["d"]))
    assert max_rel(out, g(golden, f"{name}/reduce_out")) < 1e-6


def test_gemv_matches_reference_cuda_file(case, golden):
    name, p, banks, x = case
    idx = g(golden, f"{name}/routing_indices")
    w = g(golden, f"{name}/routing_weights", BF16)
    act, out = moe.routed_decode_reference(x, idx, w, banks)
    want_act, want_out = g(golden, f"{name}/gemv_activated"), g(golden, f"{name}/gemv_out")
    assert not torch.isnan(want_out).any()
    assert max_rel(act.float(), want_act) < 8e-3
    # feed the reference's own activations so only the down projection is compared
    assert max_rel(out, want_out) < 8e-3
    assert max_rel(want_out, moe.routed_experts_fp32(x, idx, w, banks)) < 2e-2


def test_tp_shards_sum_to_whole(case):
    """Slicing per scripts/make_flashpack.py:30-35 and summing the ranks' partial
    outputs reproduces the unsharded result (float64 yard-stick)."""
    name, p, banks, x = case
    c = cases.LAYER_CASES[name]
    idx = torch.stack([torch.randperm(c["experts"])[: c["top_k"]] for _ in range(x.shape[0])])
    w = torch.rand(x.shape[0], c["top_k"]).to(BF16)
    whole = moe.routed_experts_fp32(x, idx, w, banks)
    for world in (2, 4):
        if (c["f"] // world) % 16:
            continue
        parts = sum(moe.routed_experts_fp32(x, idx, w, {e: moe.shard_banks(b, r, world) for e, b in banks.items()})
                    for r in range(world))
        assert max_rel(parts, whole) < 1e-9


# ------------------------------------------------------------------------ glue
def _bf16_ulps(a, b):
    a = a.to(BF16).view(torch.int16).to(torch.int32)
    b = b.to(BF16).view(torch.int16).to(torch.int32)
    a = torch.where(a < 0, -(a & 0x7FFF), a)
    b = torch.where(b < 0, -(b & 0x7FFF), b)
    return (a - b).abs()


def test_rms_norm_matches_reference_module_and_triton_kernel(golden):
    gen = torch.Generator().manual_seed(cases.GLUE_SEED)
    x, w = cases.glue_inputs(gen)
    got = moe.rms_norm_reference(x, w, cases.EPS)
    assert torch.equal(got.float(), g(golden, "glue/norm_bf16"))          # the reference's own CPU arithmetic
    got32 = moe.rms_norm_reference(x.float(), w.float(), cases.EPS)
    assert max_rel(got32, g(golden, "glue/norm_triton_fp32")) < 1e-6


def test_short_conv_matches_reference_module_and_triton_kernel(golden):
    gen = torch.Generator().manual_seed(cases.GLUE_SEED)
    cases.glue_inputs(gen)
    seq, taps, res = cases.sconv_inputs(gen)
    k = taps.shape[-1]
    history = torch.zeros(seq.shape[0], seq.shape[-1], k)
    history[..., 1:] = seq[:, : k - 1].float().transpose(1, 2)
    y, new_history = moe.short_conv_reference(seq[:, -1], taps, history, res[:, -1])
    # the module's convolution sums its taps in another order: a BF16 ulp on a few channels at most
    ulps = _bf16_ulps(y, g(golden, "glue/sconv_module_bf16"))
    assert int(ulps.max()) <= 1 and float((ulps > 0).float().mean()) < 0.02
    y0, _ = moe.short_conv_reference(seq[:, -1], taps, history, None)
    ulps = _bf16_ulps(y0, g(golden, "glue/sconv_module_bf16_no_residual"))
    assert int(ulps.max()) <= 1 and float((ulps > 0).float().mean()) < 0.02
    # FP32 run of the Triton kernel: same taps, same order, same history update
    y32, h32 = moe.short_conv_reference(seq[:, -1].float(), taps, history, res[:, -1].float())
    assert max_rel(y32, g(golden, "glue/sconv_triton_fp32")) < 1e-6
    assert torch.equal(h32, g(golden, "glue/sconv_triton_history"))
    assert torch.equal(new_history, h32)


def test_stack_of_blocks_matches_reference_modules(golden):
    blocks = [cases.make_layer(**c) for c in cases.stack_cases()]
    x = blocks[0][2][:1]
    weight = cases.stack_norm_weight(x.shape[-1])
    got = moe.stack_reference(x, [(p, banks) for p, banks, _ in blocks], weight, cases.EPS)
    for i in range(len(blocks)):
        want_idx = g(golden, f"stack/{i}/indices")
        assert torch.equal(got["routing"][i][0].sort().values, want_idx.sort().values), i
        assert max_rel(got["moe_out"][i].float(), g(golden, f"stack/{i}/moe_out")) < 1e-2
    assert max_rel(got["residual"].float(), g(golden, f"stack/{len(blocks) - 1}/residual")) < 1e-2
    assert max_rel(got["normed"].float(), g(golden, f"stack/{len(blocks) - 1}/normed")) < 1e-2
    # and the float64 yard-stick driven by the reference's routing stays within the bar of it
    routing = []
    n = x.clone()
    h = x.clone()
    for i, (p, banks, _) in enumerate(blocks):
        _, w, idx, gam = moe.router(n, p["router_weight"], p["router_bias"], p["global_scale"], p["route_scale"],
                                    p["top_k"], p["n_shared"])
        routing.append((idx, w, gam))
        m = moe.moe_layer_fp32(n, p, banks, idx, w, gam).float()
        h, n = moe.add_rms_norm_reference(m, h, weight, cases.EPS)
    fp_n, fp_h = moe.stack_fp32(x, [(p, banks) for p, banks, _ in blocks], weight, cases.EPS, routing)
    assert max_rel(fp_n.float(), g(golden, f"stack/{len(blocks) - 1}/normed")) < 2e-2
    assert max_rel(fp_h.float(), g(golden, f"stack/{len(blocks) - 1}/residual")) < 2e-2


@pytest.mark.parametrize("name", ["tiny", "small"])
def test_bf16_bank_gemv_matches_reference_cuda_file(golden, name):
    c = cases.LAYER_CASES[name]
    p, banks, x = cases.make_layer(**c)
    bf = cases.bf16_banks(banks)
    idx = g(golden, f"{name}/router_indices")
    w = g(golden, f"{name}/router_weights", BF16)
    act, out = moe.routed_decode_bf16_reference(x, idx, w, bf)
    want_act, want_out = g(golden, f"{name}/bf16_gemv_activated"), g(golden, f"{name}/bf16_gemv_out")
    assert not torch.isnan(want_out).any()
    assert max_rel(act.float(), want_act) < 8e-3
    assert max_rel(out, want_out) < 8e-3
    assert max_rel(want_out, moe.routed_experts_bf16_fp32(x, idx, w, bf)) < 2e-2
