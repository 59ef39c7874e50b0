"""Two CPU ranks over gloo: the tensor-parallel slicing every rank applies to the SAME
seeded weights, and the single all-reduce that sums the ranks' partial block outputs.
Expert arithmetic is the float64 oracle here (no GPU); what is under test is the host
logic of the N>1 path: `make_expert_banks(rank, world)`, `make_layer_params(rank, world)`
and `kernels.paired_all_reduce.all_reduce`."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _worker(rank: int, world: int, port: int, results):
    for p in (ROOT, ROOT / "tests" / "golden"):
        sys.path.insert(0, str(p))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import inkling_b200 as ib
        from inkling_b200.kernels.paired_all_reduce import all_reduce
        from oracle import moe as oracle_moe

        d, f, experts, ns, k, seed = 256, 128, 8, 2, 2, 17
        whole = ib.make_expert_banks(experts, d, f, "cpu", seed, chunk=4)
        mine = ib.make_expert_banks(experts, d, f, "cpu", seed, rank=rank, world=world, chunk=4)
        full_p = ib.make_layer_params(d, f, experts, ns, "cpu", seed)
        my_p = ib.make_layer_params(d, f, experts, ns, "cpu", seed, rank=rank, world=world)
        # every rank cut its slice out of the same weights, the way the reference shards a checkpoint
        for e in range(experts):
            want = oracle_moe.shard_banks(whole.weights[e], rank, world)
            for name, t in mine.weights[e].items():
                assert torch.equal(t, want[name]), (e, name)
        sg, su, sd = oracle_moe.shard_shared(full_p["shared_gate"], full_p["shared_up"], full_p["shared_down"], rank, world)
        assert torch.equal(my_p["shared_gate"], sg) and torch.equal(my_p["shared_up"], su) and torch.equal(my_p["shared_down"], sd)
        assert torch.equal(my_p["router_weight"], full_p["router_weight"])   # router replicated
        gen = torch.Generator().manual_seed(3)
        x = torch.randn(3, d, generator=gen).to(torch.bfloat16)
        idx = torch.stack([torch.randperm(experts, generator=gen)[:k] for _ in range(3)])
        w = torch.rand(3, k, generator=gen).to(torch.bfloat16)
        gam = torch.rand(3, ns, generator=gen).to(torch.bfloat16)
        partial = oracle_moe.routed_experts_fp32(x, idx, w, mine.weights) + oracle_moe.shared_experts_fp32(
            x, gam, my_p["shared_gate"], my_p["shared_up"], my_p["shared_down"])
        partial = partial.float()
        total = all_reduce(partial, dist.group.WORLD)           # the one collective of the block
        assert total.data_ptr() == partial.data_ptr()           # reduced in place, tensor returned
        want = oracle_moe.routed_experts_fp32(x, idx, w, whole.weights) + oracle_moe.shared_experts_fp32(
            x, gam, full_p["shared_gate"], full_p["shared_up"], full_p["shared_down"])
        err = float((total.double() - want).abs().max() / want.abs().max())
        results[rank] = err
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_ranks_slice_the_same_weights_and_sum_to_the_whole(world):
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = 29600 + os.getpid() % 200
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert len(results) == world and all(err < 1e-6 for err in results.values()), dict(results)


def test_all_reduce_without_a_process_group_is_the_identity():
    from inkling_b200.kernels.paired_all_reduce import all_reduce

    x = torch.arange(8, dtype=torch.float32)
    assert all_reduce(x, None) is x
