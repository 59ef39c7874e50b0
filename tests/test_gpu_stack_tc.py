"""GPU parity of the tensor-core variant of the one-launch stack kernel
(INKLING_STACK_TENSOR_CORES=1: the routed experts' packed NVFP4 banks feed
tcgen05.mma.kind::mxf4nvf4 directly, activations as E2M1 digit rows): one block against the
CPU oracle at the full shapes, stacks against the launch-by-launch path and against the
CUDA-core variant of the same kernel, run-to-run determinism and graph replay."""
import pytest
import torch

from helpers import BF16, assert_router_matches, max_rel
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


@pytest.fixture()
def tensor_cores(monkeypatch):
    monkeypatch.setenv("INKLING_STACK_TENSOR_CORES", "1")


def test_full_shape_block_against_oracle(ib, device, tensor_cores):
    d, f, E, ns, k = 4096, 2048, 64, 2, 6
    banks = ib.make_expert_banks(E, d, f, device, seed=0)
    lp = ib.make_layer_params(d, f, E, ns, device, seed=0)
    experts = ib.ResidentExperts(d, f, None, banks.weights)
    layer = ib.FusedMoE(lp["router_weight"], lp["router_bias"], lp["global_scale"], 8.0, k, lp["shared_gate"],
                        lp["shared_up"], lp["shared_down"], experts, None)
    gen = torch.Generator().manual_seed(123)
    for _ in range(2):   # the second launch runs on counters the first one left behind
        x = torch.randn(1, d, generator=gen).to(BF16)
        out = layer(x.to(device).unsqueeze(0))[0]
        torch.cuda.synchronize()
        assert layer._fused.bank_maps is not None, "the tensor-core variant did not engage"
        layer._fused.check_status()
        idx, w, gam = layer.topk_indices[:1].cpu(), layer.topk_weights[:1].cpu(), layer.gammas[:1].cpu()
        p = {key: (v.cpu() if isinstance(v, torch.Tensor) else v) for key, v in lp.items()}
        p.update(experts=E, n_shared=ns, top_k=k, route_scale=8.0)
        assert_router_matches(p, x, idx, w, gam)
        cpu_banks = {int(e): {n: t.cpu() for n, t in banks.weights[int(e)].items()} for e in idx.flatten()}
        assert max_rel(out.float(), oracle_moe.moe_layer_fp32(x, p, cpu_banks, idx, w, gam)) <= TOL


@pytest.mark.parametrize("shape", [(3, 1024, 512, 32), (2, 2048, 256, 32), (2, 4096, 256, 32), (2, 4096, 512, 32),
                                   (2, 4096, 1024, 32), (2, 4096, 2048, 32)])
def test_stack_against_launch_by_launch_and_cuda_cores(ib, device, monkeypatch, shape):
    n_layers, d, f, experts = shape
    gen = torch.Generator().manual_seed(9)
    x = torch.randn(1, d, generator=gen).to(BF16).to(device)

    def run(tensor_cores: bool):
        monkeypatch.setenv("INKLING_STACK_TENSOR_CORES", "1" if tensor_cores else "0")
        stack = ib.MoEStack.synthetic(n_layers, d, f, experts, 2, 6, device, seed=3, bias_std=0.05)
        first = stack(x).clone()
        second = stack(x).clone()
        torch.cuda.synchronize()
        stack._fused.check_status()
        assert (stack._fused.bank_maps is not None) == tensor_cores
        assert torch.equal(first, second)   # same bits run to run: parts of a tile are added in a fixed order
        return stack, first

    stack, fused = run(True)
    _, cuda_cores = run(False)
    stack.one_launch = False
    plain = stack(x).clone()
    torch.cuda.synchronize()
    assert torch.isfinite(fused.float()).all()
    assert max_rel(fused.float(), plain.float()) <= TOL
    assert max_rel(fused.float(), cuda_cores.float()) <= TOL


def test_graph_replay_equals_eager(ib, device, tensor_cores):
    stack = ib.MoEStack.synthetic(4, 1024, 512, 32, 2, 6, device, seed=5, bias_std=0.05)
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
    assert stack._fused.bank_maps is not None
    stack._fused.check_status()
