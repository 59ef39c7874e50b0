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
