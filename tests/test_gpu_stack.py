"""GPU parity of the one-launch stack kernel (ink_moe_stack_decode): one block against
the CPU oracle, a stack of blocks against the same blocks run launch by launch, and
CUDA-graph replay against eager execution."""
import pytest
import torch

import cases
from helpers import BF16, assert_router_matches, banks_to_device, layer_on_device, max_rel
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


def build_layer(ib, device, p, banks):
    dp = layer_on_device(p, device)
    experts = ib.ResidentExperts(p["d"], p["f"], None, banks_to_device(banks, device))
    return ib.FusedMoE(dp["router_weight"], dp["router_bias"], dp["global_scale"], p["route_scale"], p["top_k"],
                       dp["shared_gate"], dp["shared_up"], dp["shared_down"], experts, None)


@pytest.mark.parametrize("name", ["mid", "tp8_slice"])
def test_one_block_one_launch_against_oracle(ib, device, name):
    c = dict(cases.LAYER_CASES[name], tokens=4)
    p, banks, x = cases.make_layer(**c)
    layer = build_layer(ib, device, p, banks)
    assert layer.one_launch_supported()
    for i in range(x.shape[0]):
        xi = x[i:i + 1]
        out = layer(xi.to(device).unsqueeze(0))[0]
        torch.cuda.synchronize()
        layer._fused.check_status()
        idx, w, gam = layer.topk_indices[:1].cpu(), layer.topk_weights[:1].cpu(), layer.gammas[:1].cpu()
        assert_router_matches(p, xi, idx, w, gam)
        assert max_rel(out.float(), oracle_moe.moe_layer_fp32(xi, p, banks, idx, w, gam)) <= TOL


def test_one_launch_agrees_with_launch_by_launch(ib, device):
    """Same block, same token: the persistent kernel against router+plan, gate/up, down
    launched one after the other (two tokens in one call take that path)."""
    p, banks, x = cases.make_layer(**dict(cases.LAYER_CASES["mid"], tokens=2))
    layer = build_layer(ib, device, p, banks)
    both = layer(x.to(device).unsqueeze(0))[0].float().cpu()
    for i in range(2):
        one = layer(x[i:i + 1].to(device).unsqueeze(0))[0].float().cpu()
        assert max_rel(one[0], both[i]) <= 4e-3   # BF16 output: at most one ulp of the largest element


def make_stack(ib, device, n_layers, d, f, experts, seed=3):
    return ib.MoEStack.synthetic(n_layers, d, f, experts, 2, 6, device, seed=seed, bias_std=0.05)


def test_stack_one_launch_against_launch_by_launch(ib, device):
    stack = make_stack(ib, device, 3, 1024, 512, 32)
    assert stack.one_launch
    gen = torch.Generator().manual_seed(9)
    x = torch.randn(1, 1024, generator=gen).to(BF16).to(device)
    fused = stack(x).clone()
    fused_residual = stack.residual[:1].clone()
    torch.cuda.synchronize()
    stack._fused.check_status()
    routing = [layer.topk_indices[:1].clone() for layer in stack.layers]
    stack.one_launch = False
    plain = stack(x).clone()
    torch.cuda.synchronize()
    stack.one_launch = True
    for layer, idx in zip(stack.layers, routing):
        assert torch.equal(layer.topk_indices[:1].sort(-1).values, idx.sort(-1).values)
    assert max_rel(fused_residual.float(), stack.residual[:1].float()) <= 8e-3
    assert max_rel(fused.float(), plain.float()) <= 1.6e-2


def test_stack_graph_replay_equals_eager(ib, device):
    stack = make_stack(ib, device, 4, 1024, 512, 32, seed=5)
    gen = torch.Generator().manual_seed(10)
    xs = torch.randn(3, 1, 1024, generator=gen).to(BF16).to(device)
    runner = ib.DecodeStackGraph(stack, xs[0])
    for i in range(3):
        runner.token_in.copy_(xs[i])
        replayed = runner.replay().clone()
        torch.cuda.synchronize()
        eager = stack(xs[i]).clone()
        torch.cuda.synchronize()
        assert torch.equal(replayed, eager)
    stack._fused.check_status()


def test_baseline_shape_stack_runs_and_is_deterministic(ib, device):
    """Two blocks at the full shapes: finite output, identical on a second run."""
    stack = make_stack(ib, device, 2, 4096, 2048, 256, seed=1)
    gen = torch.Generator().manual_seed(11)
    x = torch.randn(1, 4096, generator=gen).to(BF16).to(device)
    first = stack(x).clone()
    second = stack(x).clone()
    torch.cuda.synchronize()
    stack._fused.check_status()
    assert torch.isfinite(first.float()).all() and torch.equal(first, second)
    stack.one_launch = False
    plain = stack(x).clone()
    torch.cuda.synchronize()
    assert max_rel(first.float(), plain.float()) <= 1.6e-2


# ------------------------------------------------- the stack against the oracle, block by block
def _cpu_params(layer, top_k=6, n_shared=2):
    p = dict(router_weight=layer.router_weight.cpu(), router_bias=layer.router_bias.cpu(),
             global_scale=layer.global_scale.cpu(), shared_gate=layer.shared_gate.cpu(),
             shared_up=layer.shared_up.cpu(), shared_down=layer.shared_down.cpu())
    p.update(experts=layer.experts.local, n_shared=n_shared, top_k=top_k, route_scale=layer.route_scale)
    return p


def _cpu_banks(layer, indices):
    weights = layer.experts.banks.weights
    return {int(e): {n: t.cpu() for n, t in weights[int(e)].items()} for e in indices.flatten().tolist()}


@pytest.mark.parametrize("tensor_cores", [False, True], ids=["cuda_cores", "tensor_cores"])
def test_stack_blocks_against_oracle(ib, device, monkeypatch, tensor_cores):
    """A stack of n blocks built from the same seeds is a prefix of the stack of n + 1 blocks,
    and the kernel is deterministic: the output of the n-block stack IS the input of block
    n + 1 in the longer one. That gives every block's input and output on the device, so each
    block -- router, experts, residual add, RMS norm -- is compared with the oracle on exactly
    the bits the device fed it; the whole trajectory is compared as well."""
    monkeypatch.setenv("INKLING_STACK_TENSOR_CORES", "1" if tensor_cores else "0")
    n_blocks, d, f, E = 3, 1024, 512, 32
    gen = torch.Generator().manual_seed(21)
    x = torch.randn(1, d, generator=gen).to(BF16)
    norm_weight = (1.0 + 0.1 * torch.randn(d, generator=gen)).to(BF16)
    normed, residual, routing, stacks = [x], [x], None, []
    for n in range(1, n_blocks + 1):
        stack = make_stack(ib, device, n, d, f, E, seed=7)
        stack.norm_weight.copy_(norm_weight.to(device))
        out = stack(x.to(device)).clone()
        torch.cuda.synchronize()
        stack._fused.check_status()
        assert (stack._fused.bank_maps is not None) == tensor_cores
        normed.append(out.cpu())
        residual.append(stack.residual[:1].cpu().clone())
        if n == n_blocks:
            routing = [(l.topk_indices[:1].cpu().clone(), l.topk_weights[:1].cpu().clone(), l.gammas[:1].cpu().clone())
                       for l in stack.layers]
            blocks = [(_cpu_params(l), _cpu_banks(l, r[0])) for l, r in zip(stack.layers, routing)]
        del stack
    for i, ((p, banks), (idx, w, gam)) in enumerate(zip(blocks, routing)):
        assert_router_matches(p, normed[i], idx, w, gam)                  # on the input the device saw
        m = oracle_moe.moe_layer_fp32(normed[i], p, banks, idx, w, gam).float()
        want_res, want_norm = oracle_moe.add_rms_norm_reference(m, residual[i], norm_weight, 1e-6)
        assert max_rel(residual[i + 1].float(), want_res.float()) <= TOL, i
        assert max_rel(normed[i + 1].float(), want_norm.float()) <= TOL, i
    want_norm, want_res = oracle_moe.stack_fp32(x, blocks, norm_weight, 1e-6, routing)
    assert max_rel(normed[-1].float(), want_norm.float()) <= TOL
    assert max_rel(residual[-1].float(), want_res.float()) <= TOL


def test_launch_counts_may_wrap(ib, device):
    """The kernel's counters and tags are derived from the number of launches so far, in 32
    bits: the launches on either side of the wrap give the same bits as a fresh stack."""
    stack = make_stack(ib, device, 2, 1024, 512, 32, seed=9)
    gen = torch.Generator().manual_seed(12)
    xs = torch.randn(5, 1, 1024, generator=gen).to(BF16).to(device)
    want = [stack(xs[i]).clone() for i in range(5)]
    torch.cuda.synchronize()
    stack._fused.check_status()
    stack._fused.seed_launch_count((1 << 32) - 3)
    got = [stack(xs[i]).clone() for i in range(5)]                        # launches 2^32 - 2 ... 2^32 + 2
    torch.cuda.synchronize()
    stack._fused.check_status()
    for a, b in zip(want, got):
        assert torch.equal(a, b)


def test_wait_that_runs_out_is_reported_and_recovered(ib, device):
    """A launch told that a second rank exists, whose rows nobody ever delivers: with a wait
    limit of a millisecond the kernel gives up, returns, raises bit 1 of the status word;
    check_status() reports it and resets the scratch; the next launch is correct again.
    Nothing waits without a limit and the GPU context stays usable."""
    import ctypes

    from inkling_b200.kernels import _abi, set_wait_limit

    stack = make_stack(ib, device, 2, 1024, 512, 32, seed=9)
    gen = torch.Generator().manual_seed(13)
    x = torch.randn(1, 1024, generator=gen).to(BF16).to(device)
    good = stack(x).clone()
    torch.cuda.synchronize()
    desc = stack._fused
    desc.check_status()
    size = _abi.lib().ink_moe_stack_symmetric_bytes(2, 1024, 2)
    regions = [torch.zeros(size, dtype=torch.uint8, device=device) for _ in range(2)]
    try:
        set_wait_limit(2_000_000)
        desc.world, desc.rank = 2, 0
        desc.peer_regions = (ctypes.c_uint64 * 2)(*[r.data_ptr() for r in regions])
        stack(x)
        torch.cuda.synchronize()                                          # returns: every wait was bounded
    finally:
        desc.world, desc.rank, desc.peer_regions = 1, 0, None
        set_wait_limit(200_000_000)
    assert int(desc.status.item()) & 2
    with pytest.raises(RuntimeError, match="timed out"):
        desc.check_status()
    again = stack(x).clone()
    torch.cuda.synchronize()
    desc.check_status()
    assert torch.equal(again, good)
