"""Host side of the path: the modules that stand where the reference's expert runtime
stands.

* `ResidentExperts`  -- same constructor shape, tables and `forward(hidden, top_k_index,
  top_k_weights)` as the reference's OffloadedExperts (my_inkling/offloaded_experts.py:
  25-314), with every expert resident in HBM: no cache slots, no LRU, no copy kernel.
* `FusedMoE`         -- the whole of MyInklingMoE.forward (my_inkling/model.py:361-374)
  in two or three launches plus one all-reduce: router+plan, gate/up, down+combine.
* `apply_resident_plan` / `apply_fused_moe_plan` install them into a model the way
  apply_offload_plan does (my_inkling/offloaded_experts.py:317-340).

Everything here is capture-safe: buffers are allocated in __init__ or on first use for
a given token count, and a forward issues a fixed sequence of launches.
"""
from __future__ import annotations

import torch
from torch import nn

from .kernels import (StackDescriptor, encode_bank_maps, expert_bank_names, expert_copy, expert_gemm, expert_plan, expert_reduce,
                      moe_decode, routed_decode, router_forward, router_plan_forward, router_workspace,
                      stack_supported)
from .kernels.paired_all_reduce import all_reduce

# Up to this many tokens each route runs its own matrix-vector product
# (my_inkling/offloaded_experts.py:22).
MATVEC_TOKENS = 8


def _group_of(device_mesh):
    if device_mesh is None:
        return None
    return device_mesh.get_group() if hasattr(device_mesh, "get_group") else device_mesh


def triton_cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


def _next_pow2(n: int) -> int:
    return 1 << (max(n, 1) - 1).bit_length()


class ResidentExperts(nn.Module):
    """Drop-in for the routed-experts module with every expert's banks resident.

    `weights` is keyed by global expert id, each value the bank dictionary
    {gate_up_proj, gate_up_proj_scale, gate_up_proj_scale2, down_proj, down_proj_scale,
    down_proj_scale2} of CUDA tensors already sliced for this rank (slices of every
    expert on the FFN width), inputs replicated across ranks. With `quantized=False` the
    banks are the unquantised layer's {gate_up_proj BF16 [2f, d] (rows interleave gate and
    up), down_proj BF16 [d, f]} and the pointer table has stride 2
    (kernels/grouped_experts.py:9-22); that layer runs one matrix-vector product per route
    at every token count.
    """

    def __init__(self, hidden_dim: int, intermediate_dim: int, device_mesh, weights: dict, quantized: bool = True,
                 dtype=torch.bfloat16):
        super().__init__()
        self.device_mesh = device_mesh
        self.weights = weights  # keeps the allocations alive
        self.hidden_dim, self.intermediate_dim, self.dtype = hidden_dim, intermediate_dim, dtype
        self.quantized = bool(quantized)
        names = expert_bank_names(self.quantized)
        self.stride = len(names)
        ids = sorted(weights)
        self.start, self.local, self.max_expert = ids[0], len(ids), ids[-1]
        assert ids == list(range(self.start, self.start + self.local))
        first = weights[ids[0]]
        self.device = first[names[0]].device
        assert all(w.is_contiguous() and w.is_cuda for e in weights.values() for w in e.values())
        packed = 2 if self.quantized else 1
        assert first["gate_up_proj"].shape == (2 * intermediate_dim, hidden_dim // packed)
        assert first["down_proj"].shape == (hidden_dim, intermediate_dim // packed)
        assert first["gate_up_proj"].dtype == (torch.uint8 if self.quantized else torch.bfloat16)
        self.num_slots = 0
        i32 = dict(dtype=torch.int32, device=self.device)
        self.sources = torch.tensor([[weights[e][n].data_ptr() for n in names] for e in ids],
                                    dtype=torch.int64, device=self.device)
        # banks of one kind evenly spaced in memory (one allocation per kind, say): (address of the first,
        # byte distance) per kind, for the TMA descriptors of the one-launch kernel; otherwise None
        kinds = ("gate_up_proj", "gate_up_proj_scale", "down_proj", "down_proj_scale")
        self.bank_layout = self._even_spacing([[weights[e][n].data_ptr() for e in ids] for n in kinds],
                                              [first[n].numel() * first[n].element_size() for n in kinds]) if self.quantized else None
        # TMA descriptors of the banks for the block-scaled grouped kernel, where they are evenly spaced
        self.bank_maps = None
        if self.bank_layout is not None and hidden_dim % 256 == 0 and intermediate_dim % 256 == 0:
            self.bank_maps = encode_bank_maps(self.bank_layout, self.local, hidden_dim, intermediate_dim, self.device)
        self.resident = torch.ones(self.local, **i32)
        self.destinations = torch.zeros((0, self.stride), dtype=torch.int64, device=self.device)
        self.slot_experts = torch.full((0,), -1, **i32)
        self.ages = torch.zeros(0, **i32)
        self.clock = torch.zeros((), **i32)
        self.copy_experts = torch.empty(0, **i32)
        self.pointers = torch.zeros((self.max_expert + 1) * self.stride, dtype=torch.int64, device=self.device)
        # decode reads the table without a plan when the caller skips it: start fully active
        self.pointers.view(-1, self.stride)[self.start:self.start + self.local] = self.sources
        self.experts = torch.empty(self.local, **i32)
        self.counts = torch.empty(self.local, **i32)
        self.status = torch.zeros(1, **i32)
        self.capacity = 0

    @staticmethod
    def _even_spacing(addresses: list[list[int]], sizes: list[int]):
        layout = []
        for per_expert, size in zip(addresses, sizes):
            stride = per_expert[1] - per_expert[0] if len(per_expert) > 1 else size
            if stride < size or stride % 16 or per_expert[0] % 16:
                return None
            if any(b - a != stride for a, b in zip(per_expert, per_expert[1:])):
                return None
            layout.append((per_expert[0], stride))
        return layout

    def _reserve(self, routes: int) -> None:
        if routes <= self.capacity:
            return
        self.capacity = _next_pow2(routes)
        self.rows = torch.empty((self.local, self.capacity), dtype=torch.int32, device=self.device)
        options = dict(dtype=self.dtype, device=self.device)
        self.activated = torch.empty((self.capacity, self.intermediate_dim), **options)
        self.down = torch.empty((self.capacity, self.hidden_dim), **options)

    def _plan(self, indices) -> None:
        routes = indices.numel()
        expert_plan[(1,)](indices, self.sources, self.resident, self.destinations, self.slot_experts, self.ages,
                          self.clock, self.copy_experts, self.pointers, self.experts, self.counts, self.rows,
                          self.start, self.local, self.num_slots, self.stride, routes, self.capacity,
                          _next_pow2(self.local), 1, _next_pow2(routes), num_warps=4)
        expert_copy[(128, 0)](self.sources, self.destinations, self.copy_experts, (), self.stride, 1024, 128)

    def grouped_supported(self) -> bool:
        """The tensor-core path takes NVFP4 banks whose contraction widths are multiples of 128."""
        return self.quantized and self.hidden_dim % 128 == 0 and self.intermediate_dim % 128 == 0

    def _project(self, x, indices, weights, output) -> None:
        """GEMV per route up to MATVEC_TOKENS tokens, grouped tensor-core GEMMs above
        (my_inkling/offloaded_experts.py:224-296). `output` must be zero on entry."""
        tokens = x.shape[0]
        if tokens > MATVEC_TOKENS and self.grouped_supported():
            self._project_grouped(x, indices, weights, output)
            return
        for t0 in range(0, tokens, MATVEC_TOKENS):
            t1 = min(tokens, t0 + MATVEC_TOKENS)
            routed_decode(x[t0:t1], indices[t0:t1], weights[t0:t1], self.pointers,
                          self.activated[t0 * indices.shape[1]:], output[t0:t1], self.max_expert, self.quantized,
                          status=self.status)

    def _project_grouped(self, x, indices, weights, output) -> None:
        """Both projections as grouped tensor-core GEMMs over the plan's groups, then the weighted
        sum per token (my_inkling/offloaded_experts.py:249-296). `output` must be zero on entry."""
        tokens, routes, top_k = x.shape[0], indices.numel(), indices.shape[1]
        groups = min(routes, self.local)
        for projection, inputs, target, n, k in (
                (0, x, self.activated, 2 * self.intermediate_dim, self.hidden_dim),
                (1, self.activated, self.down, self.hidden_dim, self.intermediate_dim)):
            grid = (triton_cdiv(routes, 16), triton_cdiv(n, 64), groups)
            expert_gemm[grid](inputs, self.pointers, self.experts, self.rows, self.counts, target, self.capacity,
                              n, k, top_k, projection, True, self.stride, 16, 64, 64, status=self.status,
                              bank_maps=self.bank_maps, start=self.start)
        expert_reduce[(tokens, triton_cdiv(self.hidden_dim, 256))](
            self.down, indices, weights, self.pointers, output, self.hidden_dim, top_k, self.stride,
            self.max_expert, 256)

    def forward(self, hidden_states, top_k_index, top_k_weights):
        final = torch.zeros_like(hidden_states, dtype=torch.float32)
        self._reserve(top_k_index.numel())
        self._plan(top_k_index)
        self._project(hidden_states.contiguous(), top_k_index.contiguous(), top_k_weights.contiguous(), final)
        final = all_reduce(final, _group_of(self.device_mesh))
        return final.to(hidden_states.dtype)

    def check_status(self) -> None:
        """Host read (synchronises): raises if any call since the last check routed to an
        expert id outside [0, max_expert] (bit 0 of the status word), or if a bounded wait
        inside a streaming or grouped kernel gave up (bit 1: that call's output is partial).
        Call outside graph capture."""
        flags = int(self.status.item())
        self.status.zero_()
        if flags & 2:
            raise RuntimeError("ResidentExperts: a bounded wait inside a kernel timed out; the output of that call is invalid")
        if flags & 1:
            raise RuntimeError("ResidentExperts: a route named an expert id outside the pointer table")


class FusedMoE(nn.Module):
    """Router + routed NVFP4 experts + shared BF16 experts + one all-reduce.

    Parameters are this rank's: router replicated, shared experts and routed experts
    sliced on the FFN width. forward(hidden [bs, s, d]) -> [bs, s, d] in the input dtype.
    """

    # True: one token also takes the separate launches (router + plan, gate/up, down) and the NCCL all-reduce,
    # the shape of the reference's block (my_inkling/offloaded_experts.py:298-314); used as the baseline of A/B runs
    separate_launches = False

    def __init__(self, router_weight, router_bias, global_scale, route_scale: float, top_k: int,
                 shared_gate, shared_up, shared_down, experts: ResidentExperts, device_mesh=None):
        super().__init__()
        self.router_weight, self.router_bias, self.global_scale = router_weight, router_bias.float(), global_scale
        self.route_scale, self.top_k = float(route_scale), top_k
        self.shared_gate, self.shared_up, self.shared_down = shared_gate, shared_up, shared_down
        self.n_shared = shared_gate.shape[0]
        assert experts.quantized, "FusedMoE takes NVFP4 experts; an unquantised layer keeps its own block around ResidentExperts"
        self.experts = experts
        self.device_mesh = device_mesh
        self._tokens = 0
        self._fused = None   # one-launch descriptor for a single token, built on first use

    def block_descriptor(self, norm_weight=None) -> dict:
        """This block as the one-launch kernel takes it (addresses of the module's tensors)."""
        self._reserve(1)
        ex = self.experts
        return dict(router_weight=self.router_weight, router_bias=self.router_bias, global_scale=self.global_scale,
                    sources=ex.sources, shared_gate=self.shared_gate, shared_up=self.shared_up,
                    shared_down=self.shared_down, norm_weight=norm_weight, topk_indices=self.topk_indices,
                    topk_weights=self.topk_weights, gammas=self.gammas, route_scale=self.route_scale,
                    bank_layout=ex.bank_layout if ex.start == 0 else None)

    def world_size(self) -> int:
        group = _group_of(self.device_mesh)
        if group is not None and torch.distributed.is_available() and torch.distributed.is_initialized():
            return torch.distributed.get_world_size(group)
        return 1

    def one_launch_supported(self) -> bool:
        """One token through this block in one persistent launch (the all-reduce, if any,
        follows as its own collective)."""
        ex = self.experts
        return ex.start == 0 and stack_supported(ex.hidden_dim, ex.intermediate_dim, ex.local, self.n_shared,
                                                 self.top_k)

    def _reserve(self, tokens: int) -> None:
        if tokens <= self._tokens:
            return
        dev, bf = self.router_weight.device, torch.bfloat16
        self._tokens = tokens
        self._fused = None          # descriptors hold addresses of the buffers replaced below
        self.generation = getattr(self, "generation", 0) + 1
        self.topk_weights = torch.empty(tokens, self.top_k, dtype=bf, device=dev)
        self.topk_indices = torch.empty(tokens, self.top_k, dtype=torch.int64, device=dev)
        self.gammas = torch.empty(tokens, self.n_shared, dtype=bf, device=dev)
        self.shared_activated = torch.empty(tokens * self.n_shared, self.experts.intermediate_dim, dtype=bf, device=dev)
        self.workspace = router_workspace(tokens, self.router_weight.shape[0], dev)
        self.partial = torch.empty(tokens, self.experts.hidden_dim, dtype=torch.float32, device=dev)
        self.experts._reserve(tokens * self.top_k)

    def route(self, flat):
        """Router and plan for `flat` [t, d]; fills the module's routing buffers."""
        t = flat.shape[0]
        ex = self.experts
        args = (flat, self.router_weight, self.router_bias, self.global_scale, self.route_scale, self.top_k,
                self.n_shared, self.topk_weights[:t], self.topk_indices[:t], self.gammas[:t], self.workspace)
        if t * self.top_k <= 512:
            router_plan_forward(*args, ex.sources, ex.pointers, ex.experts, ex.counts, ex.rows, ex.start,
                                ex.local, ex.stride, ex.capacity)
        else:
            router_forward(*args)
            ex._plan(self.topk_indices[:t])

    def forward(self, hidden_states):
        shape = hidden_states.shape
        flat = hidden_states.reshape(-1, shape[-1]).contiguous()
        return self.forward_partial(flat).to(hidden_states.dtype).view(shape)

    def forward_partial(self, flat):
        """flat BF16 [t, d] -> the all-reduced FP32 layer output [t, d] (a view of the
        module's own buffer, overwritten by the next call)."""
        t = flat.shape[0]
        self._reserve(t)
        ex = self.experts
        if t == 1 and self.one_launch_supported() and not self.separate_launches:
            if self._fused is None:
                # across ranks the kernel delivers and sums the partials itself: no separate collective
                self._fused = StackDescriptor([self.block_descriptor()], ex.hidden_dim, ex.intermediate_dim,
                                              ex.local, self.n_shared, self.top_k, flat.device,
                                              group=_group_of(self.device_mesh))
            self._fused.decode(flat, self.partial[:1])
            return self.partial[:1]
        self.route(flat)
        for t0 in range(0, t, MATVEC_TOKENS):
            t1 = min(t, t0 + MATVEC_TOKENS)
            moe_decode(flat[t0:t1], self.topk_indices[t0:t1], self.topk_weights[t0:t1], ex.pointers,
                       ex.activated[t0 * self.top_k:], self.shared_gate, self.shared_up, self.shared_down,
                       self.gammas[t0:t1], self.shared_activated[t0 * self.n_shared:], self.partial[t0:t1],
                       ex.max_expert, status=ex.status)
        return all_reduce(self.partial[:t], _group_of(self.device_mesh))


def apply_resident_plan(model: nn.Module, device_mesh, expert_state_dict: dict) -> nn.Module:
    """Replace every routed-experts module (a module with `gate_up_proj`, `down_proj`,
    `hidden_dim` and `intermediate_dim`, i.e. the reference's MyInklingExperts) named in
    `expert_state_dict` by ResidentExperts over this rank's banks."""
    for name, module in list(model.named_modules()):
        if name in expert_state_dict and hasattr(module, "intermediate_dim") and hasattr(module, "hidden_dim"):
            banks = expert_state_dict[name]
            quantized = "gate_up_proj_scale" in next(iter(banks.values()))   # offloaded_experts.py:333
            model.set_submodule(name, ResidentExperts(module.hidden_dim, module.intermediate_dim, device_mesh,
                                                      banks, quantized))
    return model


def apply_fused_moe_plan(model: nn.Module, device_mesh, expert_state_dict: dict) -> nn.Module:
    """Replace every MoE block (a module with `gate`, `experts` and `shared_experts`
    children, i.e. the reference's MyInklingMoE) whose experts are named in
    `expert_state_dict` by FusedMoE. The block's own router and (already sharded)
    shared-expert parameters are reused."""
    for name, module in list(model.named_modules()):
        key = name + ".experts"
        if key in expert_state_dict and all(hasattr(module, a) for a in ("gate", "experts", "shared_experts")):
            gate, shared, old = module.gate, module.shared_experts, module.experts
            experts = ResidentExperts(old.hidden_dim, old.intermediate_dim, device_mesh, expert_state_dict[key])
            fused = FusedMoE(gate.weight.data, gate.e_score_correction_bias.data, gate.global_scale.data,
                             gate.route_scale, gate.top_k, shared.gate_proj.data, shared.up_proj.data,
                             shared.down_proj.data, experts, device_mesh)
            model.set_submodule(name, fused)
    return model
