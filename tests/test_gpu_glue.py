"""GPU parity of what sits either side of the MoE block and of the unquantised expert
layer: residual add + RMS norm, the short convolution (mlp_sconv) with the decoder
residual, the BF16-bank GEMV (the reference's QUANT=0 build), against the CPU oracle and
against fixtures written by the reference's own modules and kernels."""
import pytest
import torch

import cases
from helpers import BF16, bf16_ulps, max_rel
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


def g(golden, key, dtype=None):
    t = torch.from_numpy(golden[key])
    return t.to(dtype) if dtype is not None else t


def test_add_rmsnorm_against_oracle_and_reference_module(ib, device, golden):
    gen = torch.Generator().manual_seed(cases.GLUE_SEED)
    x, w = cases.glue_inputs(gen)
    # residual = 0, partial = x: the norm of bf16(x) is the reference module's fixture
    residual = torch.zeros_like(x).to(device)
    normed = torch.empty_like(residual)
    ib.kernels.add_rmsnorm(x.float().to(device), residual, w.to(device), cases.EPS, normed)
    torch.cuda.synchronize()
    assert torch.equal(residual.cpu(), x)
    want = g(golden, "glue/norm_bf16", BF16)
    ulps = bf16_ulps(normed, want)
    assert int(ulps.max()) <= 1 and float((ulps > 0).float().mean()) < 0.01   # rsqrt and summation order: last bit
    # a real residual and an FP32 partial that does not fit BF16: both roundings of the add
    gen = torch.Generator().manual_seed(5)
    partial = torch.randn(4, 4096, generator=gen) * 0.3
    res = torch.randn(4, 4096, generator=gen).to(BF16)
    weight = (1.0 + 0.1 * torch.randn(4096, generator=gen)).to(BF16)
    want_res, want_norm = oracle_moe.add_rms_norm_reference(partial, res, weight, cases.EPS)
    res_d, norm_d = res.to(device), torch.empty(4, 4096, dtype=BF16, device=device)
    ib.kernels.add_rmsnorm(partial.to(device), res_d, weight.to(device), cases.EPS, norm_d)
    torch.cuda.synchronize()
    assert torch.equal(res_d.cpu(), want_res)                       # the BF16 add is exact arithmetic + one rounding
    ulps = bf16_ulps(norm_d, want_norm)
    assert int(ulps.max()) <= 1 and float((ulps > 0).float().mean()) < 0.01


def test_short_conv_against_oracle_and_reference(ib, device, golden):
    gen = torch.Generator().manual_seed(cases.GLUE_SEED)
    cases.glue_inputs(gen)
    seq, taps, res = cases.sconv_inputs(gen)
    k = taps.shape[-1]
    history = torch.zeros(seq.shape[0], seq.shape[-1], k)
    history[..., 1:] = seq[:, : k - 1].float().transpose(1, 2)
    want, want_history = oracle_moe.short_conv_reference(seq[:, -1], taps, history, res[:, -1])
    weight = taps.unsqueeze(1).contiguous().to(device)
    h_d = history.to(device)
    y = ib.kernels.short_conv(seq[:, -1:].contiguous().to(device), weight, h_d, res[:, -1:].contiguous().to(device))
    torch.cuda.synchronize()
    assert torch.equal(y[:, 0].cpu(), want)                         # same FP32 operations in the same order
    assert torch.equal(h_d.cpu(), want_history)
    ulps = bf16_ulps(y[:, 0], g(golden, "glue/sconv_module_bf16", BF16))
    assert int(ulps.max()) <= 1 and float((ulps > 0).float().mean()) < 0.02   # the module's conv1d sums in another order
    # without the decoder residual
    h_d = history.to(device)
    y = ib.kernels.short_conv(seq[:, -1:].contiguous().to(device), weight, h_d, None)
    want0, _ = oracle_moe.short_conv_reference(seq[:, -1], taps, history, None)
    assert torch.equal(y[:, 0].cpu(), want0)
    # FP32 input (the block's all-reduced output): rounded to BF16 first
    h_d = history.to(device)
    x32 = seq[:, -1:].float() * 1.001
    y = ib.kernels.short_conv(x32.contiguous().to(device), weight, h_d, res[:, -1:].contiguous().to(device))
    want32, want_h32 = oracle_moe.short_conv_reference(x32[:, 0].to(BF16), taps, history, res[:, -1])
    torch.cuda.synchronize()
    assert torch.equal(y[:, 0].cpu(), want32) and torch.equal(h_d.cpu(), want_h32)
    # four decode steps in a row: the history carries
    h_d, h_cpu = history.to(device), history.clone()
    for step in range(4):
        xs = torch.randn(seq.shape[0], 1, seq.shape[-1], generator=gen).to(BF16)
        y = ib.kernels.short_conv(xs.to(device), weight, h_d, None)
        want_y, h_cpu = oracle_moe.short_conv_reference(xs[:, 0], taps, h_cpu, None)
        assert torch.equal(y[:, 0].cpu(), want_y)
    assert torch.equal(h_d.cpu(), h_cpu)


def _bf16_table(dev_banks, device):
    n = max(dev_banks) + 1
    table = torch.zeros(n, 2, dtype=torch.int64)
    for e, b in dev_banks.items():
        table[e] = torch.tensor([b["gate_up_proj"].data_ptr(), b["down_proj"].data_ptr()])
    return table.reshape(-1).to(device)


@pytest.mark.parametrize("name", ["tiny", "small", "mid"])
def test_bf16_bank_gemv_against_oracle_and_reference_cuda_file(ib, device, golden, name):
    c = cases.LAYER_CASES[name]
    p, banks, x = cases.make_layer(**c)
    bf = cases.bf16_banks(banks)
    if f"{name}/bf16_gemv_out" in golden:
        idx = g(golden, f"{name}/router_indices")
        w = g(golden, f"{name}/router_weights", BF16)
    else:
        gen = torch.Generator().manual_seed(3)
        idx = torch.stack([torch.randperm(c["experts"], generator=gen)[: c["top_k"]] for _ in range(x.shape[0])])
        w = torch.rand(x.shape[0], c["top_k"], generator=gen).to(BF16)
    dev = {e: {n: t.to(device).contiguous() for n, t in b.items()} for e, b in bf.items()}
    pointers = _bf16_table(dev, device)
    t, k = idx.shape
    activated = torch.zeros(t * k, c["f"], dtype=BF16, device=device)
    out = torch.full((t, c["d"]), float("nan"), dtype=torch.float32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    ib.kernels.routed_decode(x.to(device), idx.to(device), w.to(device), pointers, activated, out, c["experts"] - 1,
                             False, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want_act, want_out = oracle_moe.routed_decode_bf16_reference(x, idx, w, bf)
    assert max_rel(activated.cpu().float(), want_act.float()) <= 8e-3
    assert max_rel(out.cpu(), want_out) <= 8e-3
    assert max_rel(out.cpu(), oracle_moe.routed_experts_bf16_fp32(x, idx, w, bf)) <= TOL
    if f"{name}/bf16_gemv_out" in golden:
        assert max_rel(activated.cpu().float(), g(golden, f"{name}/bf16_gemv_activated")) <= 8e-3
        assert max_rel(out.cpu(), g(golden, f"{name}/bf16_gemv_out")) <= 8e-3


def test_bf16_banks_skip_inactive_and_flag_out_of_range(ib, device):
    c = cases.LAYER_CASES["small"]
    p, banks, x = cases.make_layer(**c)
    bf = cases.bf16_banks(banks)
    dev = {e: {n: t.to(device).contiguous() for n, t in b.items()} for e, b in bf.items()}
    pointers = _bf16_table(dev, device)
    pointers.view(-1, 2)[3] = 0                                      # expert 3 is "not on this rank"
    idx = torch.tensor([[3, 1, 2, 4, 5, 6], [0, 1, 2, 3, 99, 5], [7, 8, 9, 10, 11, 12]])
    w = torch.full((3, 6), 0.25).to(BF16)
    activated = torch.zeros(18, c["f"], dtype=BF16, device=device)
    out = torch.empty(3, c["d"], dtype=torch.float32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    ib.kernels.routed_decode(x.to(device), idx.to(device), w.to(device), pointers, activated, out, c["experts"] - 1,
                             False, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & 1
    kept = {e: b for e, b in bf.items() if e != 3}
    _, want = oracle_moe.routed_decode_bf16_reference(x, idx, w, kept, max_expert=c["experts"] - 1)
    assert max_rel(out.cpu(), want) <= 8e-3


def test_resident_experts_over_bf16_banks(ib, device):
    """The unquantised expert layer through the drop-in module (stride-2 pointer table), at
    more tokens than one GEMV batch."""
    c = dict(cases.LAYER_CASES["small"], tokens=11)
    p, banks, x = cases.make_layer(**c)
    bf = cases.bf16_banks(banks)
    dev = {e: {n: t.to(device).contiguous() for n, t in b.items()} for e, b in bf.items()}
    experts = ib.ResidentExperts(c["d"], c["f"], None, dev, quantized=False)
    assert experts.stride == 2
    gen = torch.Generator().manual_seed(8)
    idx = torch.stack([torch.randperm(c["experts"], generator=gen)[: c["top_k"]] for _ in range(11)])
    w = torch.rand(11, c["top_k"], generator=gen).to(BF16)
    out = experts(x.to(device), idx.to(device), w.to(device))
    torch.cuda.synchronize()
    experts.check_status()
    assert out.dtype == BF16
    assert max_rel(out.float(), oracle_moe.routed_experts_bf16_fp32(x, idx, w, bf)) <= TOL
