"""Several GPUs, one process each: the one-launch stack kernel with the all-reduce done
inside the kernel (tagged 8-byte stores into the other ranks' memory, bounded polls of
its own), against the same stack on one GPU, at 2, 4 and 8 ranks; and the path for more
than one token, whose per-block all-reduce is an NCCL collective. Cases that need more
GPUs than are visible are skipped."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
SHAPE = dict(n_layers=3, hidden=4096, intermediate=2048, experts=32, n_shared=2, top_k=6)
TOKENS = 5          # the more-than-one-token case


def _inputs(device):
    gen = torch.Generator().manual_seed(4)
    one = torch.randn(3, 1, SHAPE["hidden"], generator=gen).to(torch.bfloat16).to(device)
    many = torch.randn(TOKENS, SHAPE["hidden"], generator=gen).to(torch.bfloat16).to(device)
    return one, many


def _run(ib, device, mesh, rank, world):
    c = SHAPE
    stack = ib.MoEStack.synthetic(c["n_layers"], c["hidden"], c["intermediate"], c["experts"], c["n_shared"],
                                  c["top_k"], device, seed=11, device_mesh=mesh, rank=rank, world=world, bias_std=0.05)
    assert stack.one_launch
    one, many = _inputs(device)
    outs = []
    for i in range(3):                       # several launches: counters and tags carry over from one to the next
        outs.append(stack(one[i]).float().cpu().clone())
    torch.cuda.synchronize()
    stack._fused.check_status()
    routing = [layer.topk_indices[:1].cpu().clone() for layer in stack.layers]
    batch = stack(many).float().cpu().clone()            # launch-by-launch kernels + one NCCL all-reduce per block
    torch.cuda.synchronize()
    return stack, torch.stack(outs), routing, batch


def _worker(rank: int, world: int, port: int, results, tensor_cores: bool):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      INKLING_STACK_TENSOR_CORES="1" if tensor_cores else "0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        import inkling_b200 as ib

        stack, outs, routing, batch = _run(ib, device, dist.group.WORLD, rank, world)
        assert (stack._fused.bank_maps is not None) == tensor_cores
        results[rank] = (outs, routing, batch)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,tensor_cores", [(2, False), (2, True), (4, False), (8, False)],
                         ids=["2-cuda_cores", "2-tensor_cores", "4-cuda_cores", "8-cuda_cores"])
def test_ranks_match_one_gpu(world, tensor_cores, monkeypatch):
    monkeypatch.setenv("INKLING_STACK_TENSOR_CORES", "0")   # the one-GPU stack it is compared with: the default variant
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    sys.path.insert(0, str(ROOT))
    import inkling_b200 as ib

    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = 29700 + os.getpid() % 200 + 7 * world + int(tensor_cores)
    procs = [ctx.Process(target=_worker, args=(r, world, port, results, tensor_cores)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    device = torch.device("cuda", 0)
    _, want, want_routing, want_batch = _run(ib, device, None, 0, 1)
    out0, routing0, batch0 = results[0]
    for r in range(1, world):
        out, routing, batch = results[r]
        assert torch.equal(out0, out), f"ranks 0 and {r} must end with the same bits"
        assert torch.equal(batch0, batch), f"ranks 0 and {r}: NCCL path"
        for a, b in zip(routing0, routing):
            assert torch.equal(a, b)
    err = float((out0.double() - want.double()).abs().max() / want.double().abs().max())
    assert err <= 2e-2, err
    err = float((batch0.double() - want_batch.double()).abs().max() / want_batch.double().abs().max())
    assert err <= 2e-2, err
