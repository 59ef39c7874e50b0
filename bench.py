"""Decode throughput of a stack of NVFP4 MoE layers at conc=1 on 1..8 B200.

    python bench.py --gpus 1 --steps 50 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 50 --warmup 5
    python bench.py --impl reference --steps 10 --warmup 3      # CPU arm (the oracle port)

A step is one decode token through `--layers` (default 40) MoE blocks of the Inkling-Small
shape (hidden 4096; 256 NVFP4 experts of width 2048, top-6; 2 shared BF16 experts; router
258 x 4096) under CUDA-graph replay, experts sharded tensor-parallel on the FFN width. The
whole stack is ONE persistent kernel launch per token and rank; with several ranks the
all-reduce of every block happens inside that kernel (each rank stores its FP32 partial rows
as tagged 8-byte words into the other ranks' memory over NVLink and sums what it receives
in rank order): no NCCL call is in the timed region. Weights are seeded synthetic N(0, 0.02)
quantised to NVFP4 (no checkpoint offline); every step gets a fresh N(0, 1) activation
vector, and the 7.5 GB of weights a step streams are far larger than the 126 MB L2. Outside
the timed region the run checks itself (`parity` in the JSON line): every rank ends with the
same bits, a two-block stack sliced across the ranks agrees with the same two blocks on one
GPU, and no wait inside the kernel timed out. Prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (ROOT, ROOT / "tests" / "golden"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

HIDDEN, INTERMEDIATE, EXPERTS, N_SHARED, TOP_K = 4096, 2048, 256, 2, 6
METRIC, UNIT = "decode_tokens_per_s_conc1", "tok/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one moe_stack_kernel<4096,2048> launch over two
# blocks, per block (ncu; the summary sits in profiles/)
STACK_DRAM_BYTES_PER_LAYER = 189_630_000


def layer_bytes(world: int) -> dict:
    """Algorithmic bytes one rank streams per block per token."""
    f = INTERMEDIATE // world
    gate_up_routed = TOP_K * (2 * f * HIDDEN // 2 + 2 * f * HIDDEN // 16)
    gate_up_shared = N_SHARED * 2 * f * HIDDEN * 2
    down_routed = TOP_K * (HIDDEN * f // 2 + HIDDEN * f // 16)
    down_shared = N_SHARED * HIDDEN * f * 2
    router = (EXPERTS + N_SHARED) * HIDDEN * 2
    return dict(gate_up=gate_up_routed + gate_up_shared, down=down_routed + down_shared, router=router,
                total=gate_up_routed + gate_up_shared + down_routed + down_shared + router + 2 * TOP_K * 4)


def resident_bytes_per_layer(world: int) -> int:
    f = INTERMEDIATE // world
    expert = 2 * f * HIDDEN // 2 + 2 * f * HIDDEN // 16 + HIDDEN * f // 2 + HIDDEN * f // 16 + 8
    return EXPERTS * expert + N_SHARED * 3 * f * HIDDEN * 2 + (EXPERTS + N_SHARED) * HIDDEN * 2


def load_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """nvidia-smi sampled every 200 ms while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(gpu_index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            pass

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [line.split(", ") for line in Path(self.file.name).read_text().splitlines() if line.strip()]
        os.unlink(self.file.name)
        clocks, reasons, sm_max, power = [], set(), None, []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for row in rows:
            try:
                clocks.append(float(row[1]))
                sm_max = float(row[2])
                power.append(float(row[3]))
            except (ValueError, IndexError):
                continue
            for name, value in zip(names, row[5:9]):
                if value.strip().lower() == "active":
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": sm_max,
                "power_w_max": max(power) if power else None, "samples": len(clocks), "reasons": sorted(reasons)}


# ---------------------------------------------------------------- CPU arm
def cpu_layer_inputs(seed: int, pool: int = 8):
    """config[0] on the CPU: router, shared experts and a pool of `pool` NVFP4 experts
    (the router bias confines the top-6 to the pool, so only those are generated)."""
    import torch

    import cases

    gen = torch.Generator().manual_seed(seed)
    p = dict(d=HIDDEN, f=INTERMEDIATE, experts=EXPERTS, n_shared=N_SHARED, top_k=TOP_K, route_scale=8.0)
    p["router_weight"] = (torch.randn(EXPERTS + N_SHARED, HIDDEN, generator=gen) * 0.02).to(torch.bfloat16)
    bias = torch.full((EXPERTS,), -10.0)
    bias[:pool] = 0
    p["router_bias"] = bias
    p["global_scale"] = torch.ones(1, dtype=torch.bfloat16)
    for name, shape in (("shared_gate", (N_SHARED, INTERMEDIATE, HIDDEN)), ("shared_up", (N_SHARED, INTERMEDIATE, HIDDEN)),
                        ("shared_down", (N_SHARED, HIDDEN, INTERMEDIATE))):
        p[name] = (torch.randn(*shape, generator=gen) * 0.02).to(torch.bfloat16)
    banks = cases.make_expert_banks(gen, pool, HIDDEN, INTERMEDIATE)
    return p, banks, gen


def time_cpu_layer(runs: int, warmup: int, seed: int = 0):
    """Median seconds of one MoE block on the host cores through the oracle's restatement
    of the reference's PyTorch dequant+matmul path (scripts/run_naive.py:86-108 with
    my_inkling/model.py:192-226,311-350)."""
    import torch

    from oracle import moe as oracle_moe

    torch.set_num_threads(os.cpu_count() or 1)
    p, banks, gen = cpu_layer_inputs(seed)
    times = []
    for i in range(warmup + runs):
        x = torch.randn(1, HIDDEN, generator=gen).to(torch.bfloat16)
        t0 = time.perf_counter()
        oracle_moe.moe_layer_reference(x, p, banks)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    times.sort()
    return times[len(times) // 2], times


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    seconds, times = time_cpu_layer(runs=args.steps, warmup=max(args.warmup, 1))
    step_ms = 1e3 * sum(times) / len(times) * args.layers
    value = 1.0 / (sum(times) / len(times) * args.layers)
    cores = os.cpu_count() or 1
    sample = (f"{args.steps} timed forwards of ONE block (config[0]) on the host, all {cores} threads; "
              f"a token is {args.layers} such blocks, so tok/s = 1 / ({args.layers} x mean block time)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4 weights, bf16 activations, fp32 accumulate",
        "data": "synthetic", "config": config_dict(args, 1),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def config_dict(args, world: int) -> dict:
    return {
        "workload": f"configs[2]: stack of {args.layers} MoE blocks, 1 decode token per step, CUDA-graph replay",
        "layers": args.layers, "hidden": HIDDEN, "moe_intermediate": INTERMEDIATE, "routed_experts": EXPERTS,
        "shared_experts": N_SHARED, "top_k": TOP_K, "tokens_per_step": 1,
        "parallelism": (f"tp{world} on the FFN width, 1 all-reduce per block done inside the one-launch kernel "
                        "(tagged peer stores over NVLink, no NCCL call per token)") if world > 1 else "tp1",
        "l2": "inputs larger than L2: each step streams 7.5 GB of weights, fresh activations per step",
    }


# ---------------------------------------------------------------- GPU arm
def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    import inkling_b200 as ib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD

    # never ask for more memory than is free: shrink the stack instead (and say so)
    free, total = torch.cuda.mem_get_info()
    layers = args.layers
    need = resident_bytes_per_layer(world)
    reserve = 14 << 30
    if layers * need > free - reserve:
        layers = max(1, int((free - reserve) // need))
    if world > 1:
        t = torch.tensor([layers], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        layers = int(t.item())
    args.layers_built = layers

    t_build = time.perf_counter()
    stack = ib.MoEStack.synthetic(layers, HIDDEN, INTERMEDIATE, EXPERTS, N_SHARED, TOP_K, device, seed=0,
                                  device_mesh=group, rank=rank, world=world)
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t_build

    n_inputs = args.steps + args.warmup
    gen = torch.Generator().manual_seed(1234)
    host_x = torch.randn(n_inputs, 1, HIDDEN, generator=gen).to(torch.bfloat16).pin_memory()
    dev_x = host_x.to(device)
    host_out = torch.empty(1, HIDDEN, dtype=torch.bfloat16).pin_memory()
    runner = ib.DecodeStackGraph(stack, dev_x[0], capture=not args.no_graph)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing
    for i in range(args.warmup):
        runner.token_in.copy_(dev_x[i])
        runner.replay()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(args.steps):
        runner.token_in.copy_(dev_x[args.warmup + i])
        runner.replay()
    stop.record()
    barrier()
    elapsed_ms = start.elapsed_time(stop)
    clocks = sampler.stop() if sampler else None
    if world > 1:
        t = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())

    # ---- end to end: pinned host activations in, result back to the host, every step
    barrier()
    start.record()
    for i in range(args.steps):
        runner.token_in.copy_(host_x[args.warmup + i], non_blocking=True)
        out = runner.replay()
        host_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()   # conc=1: the next token needs this one
    stop.record()
    barrier()
    e2e_ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    finite = bool(torch.isfinite(host_out.float()).all())
    stack._fused.check_status()   # raises if any wait inside the kernel gave up (a collective with several ranks)
    parity = self_check(ib, stack, runner, dev_x[args.warmup], device, group, rank, world)

    # ---- per-kernel durations for the roofline: the same kernel launched once per block of
    # the stack (distinct weights each time, so nothing is L2-warm), captured into a CUDA
    # graph so that the host's launch cost is not in the number, timed with events on the
    # stream that replays it
    def time_graph(fn, rounds: int = 5) -> float:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for layer in stack.layers:
                fn(layer)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for layer in stack.layers:
                fn(layer)
        times = []
        for _ in range(rounds + 1):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) / len(stack.layers))
        return sum(times[1:]) / rounds   # first replay is warm-up

    def half(which):
        def run(layer):
            ex = layer.experts
            ib.kernels.moe_decode(stack.normed[:1], layer.topk_indices[:1], layer.topk_weights[:1], ex.pointers,
                                  ex.activated, layer.shared_gate, layer.shared_up, layer.shared_down,
                                  layer.gammas[:1], layer.shared_activated, layer.partial[:1], ex.max_expert,
                                  status=ex.status, half=which)
        return run

    kernel_ms = {
        "gate_up": time_graph(half("gate_up")),
        "down": time_graph(half("down")),
        "router_plan": time_graph(lambda layer: layer.route(stack.normed[:1])),
        "add_rmsnorm": time_graph(lambda layer: ib.kernels.add_rmsnorm(
            layer.partial[:1], stack.residual[:1], stack.norm_weight, stack.eps, stack.normed[:1])),
    }
    # ---- A/B of the collective, outside the timed region, same blocks and inputs, every rank takes part: the
    # stated baseline is the reference's shape of the block (my_inkling/offloaded_experts.py:310: separate launches
    # and ONE NCCL all-reduce of the partial per block), captured in a graph like the one-launch kernel
    nccl_ms = None
    if 1 < world <= 4:   # (measured at 2 and 4 ranks; the 8-rank run is kept to the headline path)
        plain = ib.MoEStack(list(stack.layers), HIDDEN)
        plain.one_launch = False
        for layer in stack.layers:
            layer.separate_launches = True
        plain_runner = ib.DecodeStackGraph(plain, dev_x[0], capture=not args.no_graph)
        for i in range(3):
            plain_runner.token_in.copy_(dev_x[i % n_inputs])
            plain_runner.replay()
        barrier()
        ab_steps = min(args.steps, 10)
        start.record()
        for i in range(ab_steps):
            plain_runner.token_in.copy_(dev_x[(args.warmup + i) % n_inputs])
            plain_runner.replay()
        stop.record()
        barrier()
        t = torch.tensor([start.elapsed_time(stop)], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        nccl_ms = float(t.item()) / ab_steps
        for layer in stack.layers:
            layer.separate_launches = False
    barrier()
    if rank != 0:
        leave(world)
        return

    peaks, peak_kind = load_peaks()
    bytes_ = layer_bytes(world)
    tok_s = args.steps / (elapsed_ms * 1e-3)
    e2e_tok_s = args.steps / (e2e_ms * 1e-3)
    # the one kernel inside the timed region: one launch walks every block of the stack
    launch_ms = elapsed_ms / args.steps
    launch_bytes = bytes_["total"] * layers
    achieved = launch_bytes / (launch_ms * 1e-3) / 1e9

    def phase(name):
        return {"launch_ms": kernel_ms[name], "algorithmic_bytes": bytes_[name],
                "achieved_gbs": bytes_[name] / (kernel_ms[name] * 1e-3) / 1e9,
                "frac": bytes_[name] / (kernel_ms[name] * 1e-3) / 1e9 / peaks["hbm_gbs"]}

    line = {
        "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": launch_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "nvfp4 weights, bf16 activations, fp16 products with fp32 accumulation", "data": "synthetic",
        "config": config_dict(args, world),
        "e2e": {"value": e2e_tok_s, "unit": UNIT, "h2d_bytes_per_step": HIDDEN * 2, "d2h_bytes_per_step": HIDDEN * 2},
        "gpu_launches": args.steps * stack.launches_per_step(),
        "clocks": clocks,
        "roofline": {
            "bound": "hbm", "kernel": "moe_stack_kernel<4096,2048> (every block of the stack in one launch)",
            "achieved": achieved, "peak": peaks["hbm_gbs"], "peak_kind": peak_kind, "unit": "GB/s",
            "frac": achieved / peaks["hbm_gbs"],
            "traffic": STACK_DRAM_BYTES_PER_LAYER * layers if world == 1 else None,
            "traffic_note": "dram read+write of a 2-block launch under ncu, per block, times the blocks of this launch",
            "algorithmic_bytes_per_launch": launch_bytes, "launch_ms": launch_ms,
        },
        # the same path as separate launches (what the modules run for more than one token)
        "kernels": {
            "gate_up_stream_kernel": phase("gate_up"), "down_stream_kernel": phase("down"),
            "router_plan_launch_ms": kernel_ms["router_plan"], "add_rmsnorm_launch_ms": kernel_ms["add_rmsnorm"],
            "layer_bytes_per_rank": bytes_["total"],
        },
        "build_seconds": build_s, "layers_built": layers, "output_finite": finite, "parity": parity,
    }
    if layers != args.layers:
        line["config"]["workload"] += f" (only {layers} blocks fit in free device memory)"
        line["config"]["layers"] = layers
    if nccl_ms is not None:
        line["collective_ab"] = {
            "in_kernel_tagged_stores_ms_per_step": launch_ms,
            "launch_by_launch_nccl_all_reduce_ms_per_step": nccl_ms,
            "speedup": nccl_ms / launch_ms,
            "note": "same blocks, graph replay; baseline = 4 launches + one ncclAllReduce per block"}
    if world == 1:
        # configs[3] on four blocks of the same stack (outside the timed region): the grouped tensor-core path
        # against the per-route GEMV at 64 tokens
        line["batched"] = batched_numbers(ib, list(stack.layers[:4]), 3)["64"]
        line["batched"]["workload"] = "configs[3]: one block, 64 tokens, Zipf(1.1) routing, routed experts only"
    if world == 1 and not args.no_cpu_baseline:
        seconds, times = time_cpu_layer(runs=10, warmup=2)
        cores = os.cpu_count() or 1
        line["cpu_baseline"] = {
            "value": 1.0 / (seconds * layers), "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"median of 10 forwards of one block (config[0]) through the CPU oracle, {cores} threads; "
                      f"scaled to {layers} blocks per token", "block_seconds": seconds}
    print(json.dumps(line), flush=True)
    leave(world)


def self_check(ib, stack, runner, x, device, group, rank: int, world: int) -> dict:
    """Outside the timed region: (1) the output of the last replay is bit-identical on every rank
    (the replicated routers of the next block need that); (2) a two-block stack of the full shapes
    sliced across the ranks against the same blocks unsliced on rank 0 (each block on its own, on the same input,
    so that the routers see identical bits) -- with one rank: the one-launch kernel against the launch-by-launch
    kernels on the first two blocks of the stack --
    as max|a-b|/max|b| (bar 2e-2) and per element with a floor of 5 % of the largest magnitude."""
    import torch
    import torch.distributed as dist

    def errors(a, b):
        a, b = a.double().cpu(), b.double().cpu()
        floor = 0.05 * b.abs().max().clamp_min(1e-30)
        return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30)), float(((a - b).abs() / b.abs().clamp_min(floor)).max())

    runner.token_in.copy_(x)
    out = runner.replay()
    bits = out.view(torch.int16).to(torch.int64)
    checksum = (bits * torch.arange(1, bits.numel() + 1, device=device).view_as(bits)).sum().view(1)
    identical = True
    if world > 1:
        sums = [torch.zeros_like(checksum) for _ in range(world)]
        dist.all_gather(sums, checksum, group=group)
        identical = all(int(t.item()) == int(sums[0].item()) for t in sums)
        # Two different blocks, each run on its own on the same input by the sliced ranks and, on rank 0, unsliced:
        # with identical inputs the replicated routers must agree bit for bit, so only expert arithmetic differs.
        result = {"ranks_identical": identical,
                  "checked": f"2 blocks, each sliced over {world} ranks vs the same block on one GPU, same input"}
        worst, worst_floor, same_routing = 0.0, 0.0, True
        for seed in (7000, 8000):
            sliced = ib.MoEStack.synthetic(1, HIDDEN, INTERMEDIATE, EXPERTS, N_SHARED, TOP_K, device, seed=seed,
                                           device_mesh=group, rank=rank, world=world, bias_std=0.05)
            got = sliced(x).float().clone()
            torch.cuda.synchronize()
            sliced._fused.check_status()
            if rank == 0:
                whole = ib.MoEStack.synthetic(1, HIDDEN, INTERMEDIATE, EXPERTS, N_SHARED, TOP_K, device, seed=seed,
                                              bias_std=0.05)
                want = whole(x).float().clone()
                torch.cuda.synchronize()
                same_routing &= torch.equal(sliced.layers[0].topk_indices[:1], whole.layers[0].topk_indices[:1])
                a, b = errors(got, want)
                worst, worst_floor = max(worst, a), max(worst_floor, b)
                del whole
            del sliced
            dist.barrier(group)
        if rank == 0:
            result.update(max_rel=worst, max_rel_floor=worst_floor, same_routing=bool(same_routing),
                          ok=bool(identical and same_routing and worst <= 2e-2))
        return result
    first_two = ib.MoEStack(list(stack.layers[:2]), HIDDEN)
    fused = first_two(x).float().clone()
    torch.cuda.synchronize()
    first_two._fused.check_status()
    first_two.one_launch = False
    plain = first_two(x).float().clone()
    torch.cuda.synchronize()
    max_rel, max_rel_floor = errors(fused, plain)
    return {"ranks_identical": True, "checked": "first 2 blocks: one-launch kernel vs launch-by-launch kernels",
            "max_rel": max_rel, "max_rel_floor": max_rel_floor, "ok": bool(max_rel <= 2e-2)}


def batched_numbers(ib, layers, steps: int, token_counts=(64,)) -> dict:
    """configs[3]: `tokens` tokens through ONE block of the full shapes, routing skewed by Zipf(1.1), routed experts
    only: the grouped tensor-core path (block-scaled tcgen05 on the packed banks) against the per-route GEMV path on
    the same routing. `layers` are rotated so that nothing is L2-warm. Per token count: milliseconds of both paths and
    the weight bytes of the DISTINCT experts per second of the grouped path (each expert's 14 155 776 bytes once)."""
    import torch

    device = layers[0].router_weight.device
    expert_bytes = 2 * INTERMEDIATE * HIDDEN // 2 + 2 * INTERMEDIATE * HIDDEN // 16 + HIDDEN * INTERMEDIATE // 2 + HIDDEN * INTERMEDIATE // 16
    peaks, peak_kind = load_peaks()
    out = {}
    for tokens in token_counts:
        gen = torch.Generator().manual_seed(7)
        probs = 1.0 / torch.arange(1, EXPERTS + 1).float() ** 1.1
        perm = torch.randperm(EXPERTS, generator=gen)
        idx = torch.stack([perm[torch.multinomial(probs, TOP_K, replacement=False, generator=gen)] for _ in range(tokens)])
        idx = idx.to(device)
        w = torch.rand(tokens, TOP_K, generator=gen).to(torch.bfloat16).to(device)
        x = torch.randn(tokens, HIDDEN, generator=gen).to(torch.bfloat16).to(device)
        distinct = int(torch.unique(idx).numel())

        def timed(fn):
            for layer in layers:
                fn(layer)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(steps):
                for layer in layers:
                    fn(layer)
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / (steps * len(layers))

        def grouped(layer):
            ex = layer.experts
            final = torch.zeros(tokens, HIDDEN, dtype=torch.float32, device=device)
            ex._reserve(idx.numel())
            ex._plan(idx)
            ex._project_grouped(x, idx, w, final)

        def gemv(layer):
            for i in range(0, tokens, 8):
                layer.experts(x[i:i + 8], idx[i:i + 8], w[i:i + 8])

        grouped_ms, gemv_ms = timed(grouped), timed(gemv)
        out[str(tokens)] = {
            "tokens": tokens, "routes": tokens * TOP_K, "distinct_experts": distinct,
            "grouped_tcgen05_ms": grouped_ms, "gemv_per_route_ms": gemv_ms, "speedup": gemv_ms / grouped_ms,
            "grouped_weight_gbs": distinct * expert_bytes / (grouped_ms * 1e-3) / 1e9,
            "frac_of_peak": distinct * expert_bytes / (grouped_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "peak_kind": peak_kind}
    return out


def run_batched(args) -> None:
    """configs[3] on its own (not the headline metric): prints one JSON line with the sweep over token counts."""
    import torch

    import inkling_b200 as ib

    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    layers = [ib.MoEStack.synthetic(1, HIDDEN, INTERMEDIATE, EXPERTS, N_SHARED, TOP_K, device, seed=100 + i).layers[0]
              for i in range(args.batched_blocks)]
    numbers = batched_numbers(ib, layers, args.steps, token_counts=(9, 16, 32, 64))
    print(json.dumps({
        "metric": "batched_decode_block_ms", "value": numbers["64"]["grouped_tcgen05_ms"], "unit": "ms",
        "higher_is_better": False, "n_gpus": 1, "steps": args.steps, "data": "synthetic",
        "config": {"workload": "configs[3]: one block, 64 tokens, Zipf(1.1) routing, routed experts only"},
        "by_tokens": numbers}), flush=True)


def run_attention(args) -> None:
    """Decode attention on its own (not the headline metric): one token against the K/V caches of `--layers` layers
    at the model's shapes (64 heads of 128 channels; sliding layers 16 key/value heads x 512 slots, every sixth layer
    full attention with 8 key/value heads x 4096 slots), captured in one graph; the caches of all layers together
    are larger than the L2. Prints one JSON line: microseconds per layer and cache bytes per second."""
    import torch

    import inkling_b200 as ib

    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    gen = torch.Generator().manual_seed(3)
    heads, c, d_rel, batch = 64, 128, 16, 1
    layers, cache_bytes = [], 0
    for i in range(args.layers):
        full = (i + 1) % 6 == 0
        hk, slots, extent, window = (8, 4096, 1024, 0) if full else (16, 512, 512, 512)
        k = torch.randn(batch, hk, slots, c, generator=gen).to(torch.bfloat16).to(device)
        v = torch.randn(batch, hk, slots, c, generator=gen).to(torch.bfloat16).to(device)
        proj = (torch.randn(d_rel, extent, generator=gen) * 0.5).to(torch.bfloat16).to(device)
        layers.append((k, v, proj, window, 1024 if full else None))
        cache_bytes += 2 * 2 * batch * hk * c * (slots if window else 3001)   # K and V rows of the slots in use
    q = torch.randn(batch, heads, c, generator=gen).to(torch.bfloat16).to(device)
    r = torch.randn(batch, heads, d_rel, generator=gen).to(torch.bfloat16).to(device)
    news = {hk: torch.randn(batch, hk, 1, c, generator=gen).to(torch.bfloat16).to(device) for hk in (8, 16)}   # the token's key / value
    # every slot of a sliding ring is in use; a full layer has seen 3000 of its 4096 positions
    pos_sliding = torch.tensor(5000, dtype=torch.int64, device=device)
    pos_full = torch.tensor(3000, dtype=torch.int64, device=device)
    out = torch.empty(batch, heads, 1, c, dtype=torch.bfloat16, device=device)

    def step():
        for k, v, proj, window, n_floor in layers:
            position = pos_sliding if window else pos_full
            ib.kernels.decode_attention(q, r, proj, k, v, position, None, window=window, log_scaling_n_floor=n_floor, out=out,
                                        new_key=news[k.shape[1]], new_value=news[k.shape[1]])

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(args.warmup):
        graph.replay()
    torch.cuda.synchronize()
    start.record()
    for _ in range(args.steps):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / args.steps
    peaks, peak_kind = load_peaks()
    gbs = cache_bytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "decode_attention_layer_us", "value": ms * 1e3 / args.layers, "unit": "us", "higher_is_better": False,
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "data": "synthetic",
        "config": {"workload": f"decode attention (stores the token in the cache itself) of {args.layers} layers, 1 token, 64 heads x 128, sliding 16 x 512 "
                               "slots, every sixth layer full 8 x 4096 slots; graph replay", "cache_bytes_per_step": cache_bytes},
        "gpu_launches": args.layers * args.steps,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "peak_kind": peak_kind, "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "traffic": None}}), flush=True)


def leave(world: int) -> None:
    """Multi-rank runs end here, after the last barrier: tearing an NCCL communicator down while
    captured graphs still hold its kernels can block for minutes, so the ranks flush and exit."""
    if world > 1:
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--layers", type=int, default=40)
    parser.add_argument("--no-graph", action="store_true", help="eager launches instead of graph replay")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--batched", action="store_true", help="configs[3] instead of the headline workload")
    parser.add_argument("--batched-blocks", type=int, default=4, help="blocks rotated by --batched (1 for a profiler capture)")
    parser.add_argument("--attention", action="store_true", help="decode attention on its own instead of the headline workload")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.attention:
        run_attention(args)
        return
    if args.batched:
        run_batched(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
