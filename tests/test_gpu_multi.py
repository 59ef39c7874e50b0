"""Two GPUs, one process each: the one-launch stack kernel with the all-reduce done
inside the kernel (stores into the other rank's memory, bounded waits on its counter),
against the same stack on one GPU. Skipped where fewer than two GPUs are visible."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
SHAPE = dict(n_layers=2, hidden=4096, intermediate=2048, experts=64, n_shared=2, top_k=6)


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

        c = SHAPE
        stack = ib.MoEStack.synthetic(c["n_layers"], c["hidden"], c["intermediate"], c["experts"], c["n_shared"],
                                      c["top_k"], device, seed=11, device_mesh=dist.group.WORLD, rank=rank,
                                      world=world, bias_std=0.05)
        assert stack.one_launch
        gen = torch.Generator().manual_seed(4)
        xs = torch.randn(3, 1, c["hidden"], generator=gen).to(torch.bfloat16).to(device)
        outs = []
        for i in range(3):                       # several launches: the counters carry over from one to the next
            outs.append(stack(xs[i]).float().cpu().clone())
        torch.cuda.synchronize()
        stack._fused.check_status()
        assert (stack._fused.bank_maps is not None) == tensor_cores
        routing = [layer.topk_indices[:1].cpu().clone() for layer in stack.layers]
        results[rank] = (torch.stack(outs), routing)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("tensor_cores", [False, True], ids=["cuda_cores", "tensor_cores"])
def test_two_rank_stack_matches_one_gpu(tensor_cores, monkeypatch):
    monkeypatch.setenv("INKLING_STACK_TENSOR_CORES", "0")   # the one-GPU stack it is compared with: the default variant
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    sys.path.insert(0, str(ROOT))
    import inkling_b200 as ib

    c = SHAPE
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = 29700 + os.getpid() % 200
    procs = [ctx.Process(target=_worker, args=(r, 2, port + int(tensor_cores), results, tensor_cores)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0
    device = torch.device("cuda", 0)
    single = ib.MoEStack.synthetic(c["n_layers"], c["hidden"], c["intermediate"], c["experts"], c["n_shared"],
                                   c["top_k"], device, seed=11, bias_std=0.05)
    gen = torch.Generator().manual_seed(4)
    xs = torch.randn(3, 1, c["hidden"], generator=gen).to(torch.bfloat16).to(device)
    want = torch.stack([single(xs[i]).float().cpu().clone() for i in range(3)])
    out0, routing0 = results[0]
    out1, routing1 = results[1]
    assert torch.equal(out0, out1), "the ranks must end with the same bits"
    for a, b in zip(routing0, routing1):
        assert torch.equal(a, b)
    err = float((out0.double() - want.double()).abs().max() / want.double().abs().max())
    assert err <= 2e-2, err
