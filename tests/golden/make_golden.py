"""Generates tests/golden/golden.npz by RUNNING THE REFERENCE on seeded inputs.

Needs a checkout of the reference (first argument, or the environment variable
INKLING_REFERENCE_ROOT) and therefore only runs where one is mounted; the fixtures it writes
travel with the repository.

Sources, all the reference's own code:
  A. its PyTorch classes (my_inkling/model.py): MyInklingTopkRouter,
     MyInklingSharedExperts, MyInklingExperts, MyInklingMoE, on the CPU in BF16;
  B. its Triton kernels (kernels/expert_planner.py, kernels/grouped_experts.py) under
     TRITON_INTERPRET=1: expert_plan, expert_gemm (NVFP4 dequant inline), expert_reduce.
     The interpreter has no working BF16 arithmetic (its BF16 results are garbage), so
     the grouped kernels are fed FP32 activations and router weights: their
     dequantised weight tile is then the exact FP32 product, which is what pins the
     decode;
  C. its CUDA C file kernels/routed_decode.cu compiled for the CPU behind
     oracle/ref_cpu_shim.h (oracle/build_ref.py): gate_up and down_reduce, with NVFP4
     banks (QUANT=1) and with BF16 banks (QUANT=0);
  D. the glue either side of the block: MyInklingRMSNorm and MyInklingShortConv
     (my_inkling/model.py) on the CPU in BF16, their Triton twins _rms_norm and
     _short_conv (kernels/decode.py) under the interpreter in FP32, and a stack of
     three MoE blocks joined by residual add + MyInklingRMSNorm.

    python tests/golden/make_golden.py <reference_root>
"""
from __future__ import annotations

import ctypes
import os
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(HERE))
REFERENCE = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("INKLING_REFERENCE_ROOT")
if not REFERENCE:
    sys.exit("usage: make_golden.py <reference_root>  (or set INKLING_REFERENCE_ROOT)")
sys.path.insert(0, REFERENCE)

import cases  # noqa: E402
from oracle import build_ref, nvfp4  # noqa: E402

from kernels import decode as ref_decode  # noqa: E402  (reference)
from kernels.expert_planner import expert_plan  # noqa: E402  (reference)
from kernels.grouped_experts import expert_gemm, expert_reduce  # noqa: E402  (reference)
from my_inkling import model as ref_model  # noqa: E402  (reference)

BF16 = torch.bfloat16
out: dict[str, np.ndarray] = {}


def put(key: str, t) -> None:
    if isinstance(t, torch.Tensor):
        t = t.detach().cpu()
        t = t.float().numpy() if t.dtype == BF16 else t.numpy()
    out[key] = np.asarray(t)


def reference_config(c):
    return ref_model.InklingTextConfig(
        hidden_size=c["d"], vocab_size=32, num_hidden_layers=1, pad_token_id=0,
        moe_intermediate_size=c["f"], n_routed_experts=c["experts"],
        num_experts_per_tok=c["top_k"], n_shared_experts=c["n_shared"], route_scale=8.0)


@torch.no_grad()
def classes(name: str, c: dict) -> None:
    p, banks, x = cases.make_layer(**c)
    put(f"{name}/checksum", np.frombuffer(cases.layer_checksum(p, banks, x).encode(), dtype=np.uint8))
    cfg = reference_config(c)
    moe = ref_model.MyInklingMoE(cfg).bfloat16().eval()
    moe.gate.e_score_correction_bias = moe.gate.e_score_correction_bias.float()  # restore_fp32, model.py:748
    moe.gate.weight.copy_(p["router_weight"])
    moe.gate.global_scale.copy_(p["global_scale"])
    moe.gate.e_score_correction_bias.copy_(p["router_bias"])
    moe.shared_experts.gate_proj.copy_(p["shared_gate"])
    moe.shared_experts.up_proj.copy_(p["shared_up"])
    moe.shared_experts.down_proj.copy_(p["shared_down"])
    for e, b in banks.items():
        gu = nvfp4.dequant_bf16(b["gate_up_proj"], b["gate_up_proj_scale"], b["gate_up_proj_scale2"])
        # the unquantised module stores chunked halves (model.py:274-277); the checkpoint interleaves
        moe.experts.gate_up_proj[e].copy_(torch.cat([gu[0::2], gu[1::2]]))
        moe.experts.down_proj[e].copy_(nvfp4.dequant_bf16(b["down_proj"], b["down_proj_scale"], b["down_proj_scale2"]))
    hidden = x.unsqueeze(0)
    logits, w, idx, gam = moe.gate(hidden)
    put(f"{name}/router_logits", logits)
    put(f"{name}/router_weights", w)
    put(f"{name}/router_indices", idx)
    put(f"{name}/router_gammas", gam)
    put(f"{name}/shared_out", moe.shared_experts(hidden, gammas=gam)[0])
    put(f"{name}/experts_out", moe.experts(x, idx, w))
    put(f"{name}/moe_out", moe(hidden)[0])
    if name == "tiny":
        d_idx, d_w = cases.dispatch_fixture()
        put(f"{name}/dispatch_out", moe.experts(x, d_idx, d_w.to(BF16)))


def pointer_table(banks: dict, keep: list) -> torch.Tensor:
    """[experts, 6] host addresses, bank order of kernels/grouped_experts.py:9-22."""
    table = []
    for e in sorted(banks):
        row = []
        for n in cases.BANK_NAMES:
            t = banks[e][n]
            if n.endswith("scale2"):
                t = t.reshape(1).float().contiguous()
            keep.append(t)
            row.append(t.data_ptr())
        table.append(row)
    return torch.tensor(table, dtype=torch.int64)


def triton_kernels(name: str, c: dict, indices: torch.Tensor, weights: torch.Tensor) -> None:
    p, banks, x = cases.make_layer(**c)
    keep: list = []
    sources = pointer_table(banks, keep)
    E, stride, top_k = c["experts"], 6, indices.shape[1]
    routes = indices.numel()
    capacity = 1 << (routes - 1).bit_length()
    i32 = dict(dtype=torch.int32)
    pointers = torch.zeros(E * stride, dtype=torch.int64)
    experts, counts = torch.empty(E, **i32), torch.empty(E, **i32)
    rows = torch.full((E, capacity), -1, **i32)
    pow2 = lambda n: 1 << (max(n, 1) - 1).bit_length()  # noqa: E731
    expert_plan[(1,)](indices, sources, torch.ones(E, **i32), torch.zeros((0, stride), dtype=torch.int64),
                      torch.full((0,), -1, **i32), torch.zeros(0, **i32), torch.zeros((), **i32),
                      torch.empty(0, **i32), pointers, experts, counts, rows, 0, E, 0, stride, routes,
                      capacity, pow2(E), 1, pow2(routes), num_warps=4)
    put(f"{name}/plan_experts", experts)
    put(f"{name}/plan_counts", counts)
    put(f"{name}/plan_rows", rows)
    put(f"{name}/plan_active", (pointers.view(E, stride)[:, 0] != 0))
    d, f = c["d"], c["f"]
    x, weights = x.float(), weights.float()
    activated = torch.zeros(capacity, f)
    down = torch.zeros(capacity, d)
    groups = min(routes, E)
    for projection, inputs, target, n, k in ((0, x, activated, 2 * f, d), (1, activated, down, d, f)):
        grid = ((routes + 15) // 16, (n + 63) // 64, groups)
        expert_gemm[grid](inputs, pointers, experts, rows, counts, target, capacity, n, k, top_k,
                          projection, True, stride, 16, 64, 64)
    put(f"{name}/gemm_activated", activated)
    put(f"{name}/gemm_down", down)
    output = torch.zeros(x.shape[0], d, dtype=torch.float32)
    expert_reduce[(x.shape[0], (d + 255) // 256)](down, indices, weights, pointers, output, d, top_k,
                                                    stride, E - 1, 256)
    put(f"{name}/reduce_out", output)
    put(f"{name}/routing_indices", indices)
    put(f"{name}/routing_weights", weights)


def cuda_file_on_cpu(name: str, c: dict, indices: torch.Tensor, weights: torch.Tensor) -> None:
    p, banks, x = cases.make_layer(**c)
    keep: list = []
    pointers = pointer_table(banks, keep).reshape(-1).contiguous()
    d, f, top_k = c["d"], c["f"], indices.shape[1]
    tokens, routes = x.shape[0], indices.numel()
    # rows per block: the wrapper's default 16 (routed_decode.py:45), raised where a
    # block reads more rows than that per iteration (RPI = 128 / (K / 32))
    rows_up, rows_dn = max(16, 4096 // d), max(16, 4096 // f)
    activated = torch.zeros(routes, f, dtype=BF16)
    output = torch.full((tokens, d), float("nan"), dtype=torch.float32)
    flat = indices.reshape(-1).contiguous()
    lib_up = ctypes.CDLL(str(build_ref.lib_path(d, 1)))
    lib_dn = ctypes.CDLL(str(build_ref.lib_path(f, 1)))
    vp = ctypes.c_void_p
    lib_up.ref_launch_gate_up(vp(x.data_ptr()), vp(flat.data_ptr()), vp(pointers.data_ptr()),
                              vp(activated.data_ptr()), top_k, c["experts"] - 1, 2 * f, rows_up, routes)
    lib_dn.ref_launch_down_reduce(vp(activated.data_ptr()), vp(flat.data_ptr()), vp(weights.data_ptr()),
                                  vp(pointers.data_ptr()), vp(output.data_ptr()), top_k,
                                  c["experts"] - 1, d, rows_dn, tokens)
    put(f"{name}/gemv_activated", activated)
    put(f"{name}/gemv_out", output)


def load_reference_moe(c: dict, p: dict, banks: dict):
    """The reference's MyInklingMoE in BF16 holding the case's weights (NVFP4 banks
    dequantised to BF16 the way its PyTorch path does before every matmul)."""
    moe = ref_model.MyInklingMoE(reference_config(c)).bfloat16().eval()
    moe.gate.e_score_correction_bias = moe.gate.e_score_correction_bias.float()
    moe.gate.weight.copy_(p["router_weight"])
    moe.gate.global_scale.copy_(p["global_scale"])
    moe.gate.e_score_correction_bias.copy_(p["router_bias"])
    moe.shared_experts.gate_proj.copy_(p["shared_gate"])
    moe.shared_experts.up_proj.copy_(p["shared_up"])
    moe.shared_experts.down_proj.copy_(p["shared_down"])
    for e, b in banks.items():
        gu = nvfp4.dequant_bf16(b["gate_up_proj"], b["gate_up_proj_scale"], b["gate_up_proj_scale2"])
        moe.experts.gate_up_proj[e].copy_(torch.cat([gu[0::2], gu[1::2]]))
        moe.experts.down_proj[e].copy_(nvfp4.dequant_bf16(b["down_proj"], b["down_proj_scale"], b["down_proj_scale2"]))
    return moe


@torch.no_grad()
def glue() -> None:
    """Source D: norm, short convolution, and a stack of blocks."""
    gen = torch.Generator().manual_seed(cases.GLUE_SEED)
    x, w = cases.glue_inputs(gen)
    norm = ref_model.MyInklingRMSNorm(x.shape[-1], eps=cases.EPS).bfloat16()
    norm.weight.copy_(w)
    put("glue/norm_bf16", norm(x))
    put("glue/norm_triton_fp32", ref_decode.rms_norm(x.float(), w.float(), cases.EPS))
    # short convolution: the module's eager path on a sequence of K tokens pins the
    # roundings; the Triton kernel in FP32 pins the history shift and the tap order
    seq, cw, res = cases.sconv_inputs(gen)
    k = cw.shape[-1]
    conv = ref_model.MyInklingShortConv(seq.shape[-1], k, layer_idx=0, conv_idx=3)   # FP32 taps (restore_fp32)
    conv.conv1d.weight.copy_(cw.unsqueeze(1))
    put("glue/sconv_module_bf16", conv(seq, cache=None, residual=res)[:, -1])
    put("glue/sconv_module_bf16_no_residual", conv(seq, cache=None, residual=None)[:, -1])
    history = torch.zeros(seq.shape[0], seq.shape[-1], k)
    history[..., 1:] = seq[:, : k - 1].float().transpose(1, 2)
    out = ref_decode.short_conv(seq[:, -1:].float(), cw.unsqueeze(1), history, res[:, -1:].float())
    put("glue/sconv_triton_fp32", out[:, 0])
    put("glue/sconv_triton_history", history)
    # three blocks joined by residual add + norm, every module the reference's own
    blocks = [cases.make_layer(**c) for c in cases.stack_cases()]
    x = blocks[0][2][:1]
    norm = ref_model.MyInklingRMSNorm(x.shape[-1], eps=cases.EPS).bfloat16()
    norm.weight.copy_(cases.stack_norm_weight(x.shape[-1]))
    h, n = x.clone(), x.clone()
    for i, (c, (p, banks, _)) in enumerate(zip(cases.stack_cases(), blocks)):
        moe = load_reference_moe(c, p, banks)
        _, _, idx, _ = moe.gate(n.unsqueeze(0))
        m = moe(n.unsqueeze(0))[0]
        h = h + m
        n = norm(h)
        put(f"stack/{i}/indices", idx[0])
        put(f"stack/{i}/moe_out", m)
        put(f"stack/{i}/residual", h)
        put(f"stack/{i}/normed", n)


def bf16_banks_on_cpu(name: str, c: dict) -> None:
    """Source C with QUANT=0: BF16 expert banks, pointer stride 2."""
    p, banks, x = cases.make_layer(**c)
    bf = cases.bf16_banks(banks)
    idx = torch.from_numpy(out[f"{name}/router_indices"]).long().contiguous()
    w = torch.from_numpy(out[f"{name}/router_weights"]).to(BF16).contiguous()
    keep = [t for e in sorted(bf) for t in (bf[e]["gate_up_proj"], bf[e]["down_proj"])]
    pointers = torch.tensor([t.data_ptr() for t in keep], dtype=torch.int64)
    d, f, top_k = c["d"], c["f"], idx.shape[1]
    tokens, routes = x.shape[0], idx.numel()
    rows_up, rows_dn = max(32, 4096 // d), max(32, 4096 // f)   # routed_decode.py:45: 32 rows for BF16 banks
    activated = torch.zeros(routes, f, dtype=BF16)
    output = torch.full((tokens, d), float("nan"), dtype=torch.float32)
    flat = idx.reshape(-1).contiguous()
    lib_up = ctypes.CDLL(str(build_ref.lib_path(d, 0)))
    lib_dn = ctypes.CDLL(str(build_ref.lib_path(f, 0)))
    vp = ctypes.c_void_p
    lib_up.ref_launch_gate_up(vp(x.data_ptr()), vp(flat.data_ptr()), vp(pointers.data_ptr()),
                              vp(activated.data_ptr()), top_k, c["experts"] - 1, 2 * f, rows_up, routes)
    lib_dn.ref_launch_down_reduce(vp(activated.data_ptr()), vp(flat.data_ptr()), vp(w.data_ptr()),
                                  vp(pointers.data_ptr()), vp(output.data_ptr()), top_k,
                                  c["experts"] - 1, d, rows_dn, tokens)
    put(f"{name}/bf16_gemv_activated", activated)
    put(f"{name}/bf16_gemv_out", output)


def main() -> None:
    torch.manual_seed(0)
    build_ref.build(REFERENCE)
    glue()
    print("done glue", flush=True)
    for name, c in cases.LAYER_CASES.items():
        classes(name, c)
        idx = torch.from_numpy(out[f"{name}/router_indices"]).long()
        w = torch.from_numpy(out[f"{name}/router_weights"]).to(BF16)
        if name == "tiny":  # also the reference test's hand-written dispatch pattern
            idx, w = cases.dispatch_fixture()
            w = w.to(BF16)
        triton_kernels(name, c, idx.contiguous(), w.contiguous())
        cuda_file_on_cpu(name, c, idx.contiguous(), w.contiguous())
        if name in ("tiny", "small"):
            bf16_banks_on_cpu(name, c)
        print("done", name, flush=True)
    # plan-only cases: random routings incl. many routes per expert and empty experts
    gen = torch.Generator().manual_seed(99)
    for n, (E, t, k) in enumerate(((8, 1, 2), (16, 8, 6), (32, 40, 6), (256, 1, 6), (256, 64, 6))):
        idx = torch.stack([torch.randperm(E, generator=gen)[:k] for _ in range(t)])
        routes = idx.numel()
        capacity = 1 << (routes - 1).bit_length()
        sources = (torch.arange(E * 6, dtype=torch.int64).reshape(E, 6) + 1) * 256
        i32 = dict(dtype=torch.int32)
        pointers = torch.zeros(E * 6, dtype=torch.int64)
        experts, counts = torch.empty(E, **i32), torch.empty(E, **i32)
        rows = torch.full((E, capacity), -1, **i32)
        pow2 = lambda v: 1 << (max(v, 1) - 1).bit_length()  # noqa: E731
        expert_plan[(1,)](idx, sources, torch.ones(E, **i32), torch.zeros((0, 6), dtype=torch.int64),
                          torch.full((0,), -1, **i32), torch.zeros(0, **i32), torch.zeros((), **i32),
                          torch.empty(0, **i32), pointers, experts, counts, rows, 0, E, 0, 6, routes,
                          capacity, pow2(E), 1, pow2(routes), num_warps=4)
        for key, val in (("indices", idx), ("experts", experts), ("counts", counts), ("rows", rows),
                         ("pointers", pointers)):
            put(f"plan{n}/{key}", val)
        print("done plan", n, flush=True)
    np.savez_compressed(HERE / "golden.npz", **out)
    print("wrote", HERE / "golden.npz", sum(v.nbytes for v in out.values()), "bytes raw")


if __name__ == "__main__":
    main()
