"""One-launch decode of a stack of MoE blocks (ink_moe_stack_decode)."""
from __future__ import annotations

import ctypes
import os
import struct

import torch

from . import _abi

BUILT_SHAPES = {(4096, 2048), (4096, 1024), (4096, 512), (4096, 256), (2048, 256), (1024, 512)}
_LAYER_FORMAT = "<12Qfi"   # twelve pointers (the last: the banks' TMA descriptors or 0), route_scale, pad


def tensor_cores_requested() -> bool:
    """INKLING_STACK_TENSOR_CORES=1 runs the routed experts of the one-launch kernel on the tensor cores
    (tcgen05 block-scaled MMA on the packed NVFP4 banks). Off by default: the variant is parity-green but
    its per-layer staging and tile hand-over still cost more than its faster weight stream saves."""
    return os.environ.get("INKLING_STACK_TENSOR_CORES", "0") == "1"


def set_wait_limit(cycles: int) -> None:
    """SM clocks a wait inside the one-launch kernel may take before the launch gives up
    (ink_moe_stack_set_wait_limit). Default 200 000 000."""
    _abi.check(_abi.lib().ink_moe_stack_set_wait_limit(int(cycles)))


def stack_supported(hidden: int, intermediate: int, experts: int, n_shared: int, top_k: int) -> bool:
    return ((hidden, intermediate) in BUILT_SHAPES and experts <= 512 and top_k <= 8 and n_shared <= 2
            and top_k <= experts)


class StackDescriptor:
    """Device-side table of block descriptors plus the kernel's scratch; built once."""

    def __init__(self, blocks: list[dict], hidden: int, intermediate: int, experts: int, n_shared: int,
                 top_k: int, device, group=None):
        assert struct.calcsize(_LAYER_FORMAT) == _abi.lib().ink_moe_stack_layer_bytes()
        self.keep = blocks   # the tensors the addresses point into
        self.n_layers, self.hidden, self.intermediate = len(blocks), hidden, intermediate
        self.experts, self.n_shared, self.top_k = experts, n_shared, top_k
        ptr = lambda t: 0 if t is None else t.data_ptr()  # noqa: E731
        # TMA descriptors of the banks, when every block's banks are evenly spaced in memory: the routed
        # experts then run on the tensor cores
        layouts = [b.get("bank_layout") for b in blocks]
        self.bank_maps = None
        maps_at = [0] * len(blocks)
        if all(layout is not None for layout in layouts) and tensor_cores_requested():
            host = bytearray(512 * len(blocks))
            for i, layout in enumerate(layouts):
                out = (ctypes.c_char * 512).from_buffer(host, 512 * i)
                (gc, gcs), (gs, gss), (dc, dcs), (ds, dss) = layout
                _abi.check(_abi.lib().ink_moe_stack_encode_banks(out, gc, gcs, gs, gss, dc, dcs, ds, dss, experts, hidden,
                                                                 intermediate))
            self.bank_maps = torch.frombuffer(host, dtype=torch.uint8).to(device)
            assert self.bank_maps.data_ptr() % 128 == 0
            maps_at = [self.bank_maps.data_ptr() + 512 * i for i in range(len(blocks))]
        raw = b"".join(struct.pack(
            _LAYER_FORMAT, ptr(b["router_weight"]), ptr(b["router_bias"]), ptr(b["global_scale"]), ptr(b["sources"]),
            ptr(b["shared_gate"]), ptr(b["shared_up"]), ptr(b["shared_down"]), ptr(b.get("norm_weight")),
            ptr(b.get("topk_indices")), ptr(b.get("topk_weights")), ptr(b.get("gammas")), maps_at[i],
            float(b["route_scale"]), 0)
            for i, b in enumerate(blocks))
        self.table = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)
        size = _abi.lib().ink_moe_stack_scratch_bytes(self.n_layers, hidden, intermediate, experts, n_shared, top_k)
        self.scratch = torch.zeros(size, dtype=torch.uint8, device=device)   # counters start at zero, then only grow
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.rank, self.world, self.peer_regions, self.symmetric, self.group = 0, 1, None, None, None
        if group is not None and torch.distributed.is_initialized() and torch.distributed.get_world_size(group) > 1:
            self._join(group, device)

    def _join(self, group, device) -> None:
        """Tensor-parallel ranks: one symmetric buffer per rank that every rank can store into
        (torch symmetric memory does the peer mapping; this is plumbing, the kernel does the rest)."""
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.rank = torch.distributed.get_rank(group)
        self.world = torch.distributed.get_world_size(group)
        size = _abi.lib().ink_moe_stack_symmetric_bytes(self.n_layers, self.hidden, self.world)
        self.symmetric = symm_mem.empty(size, dtype=torch.uint8, device=device)
        self.symmetric.zero_()
        handle = symm_mem.rendezvous(self.symmetric, group)
        self._handle = handle
        self.peer_regions = (ctypes.c_uint64 * self.world)(*[int(p) for p in handle.buffer_ptrs])
        torch.cuda.synchronize()
        torch.distributed.barrier(group)   # every rank's region is zero before anyone delivers into it

    def decode(self, x, partial_out, residual_io=None, normed_out=None, eps: float = 1e-6) -> None:
        glue = residual_io is not None
        assert x.dtype == torch.bfloat16 and x.numel() == self.hidden and x.is_contiguous()
        assert partial_out.dtype == torch.float32 and partial_out.numel() == self.hidden
        if glue:
            assert residual_io.dtype == normed_out.dtype == torch.bfloat16
            assert residual_io.numel() == normed_out.numel() == self.hidden
        _abi.require_cuda(x, partial_out, residual_io, normed_out)
        common = (self.table.data_ptr(), self.n_layers, x.data_ptr(), _abi.ptr(residual_io), _abi.ptr(normed_out),
                  partial_out.data_ptr(), int(glue) | (2 if self.bank_maps is not None else 0), float(eps), self.hidden, self.intermediate, self.experts,
                  self.n_shared, self.top_k, self.scratch.data_ptr(), self.scratch.numel())
        if self.world == 1:
            _abi.check(_abi.lib().ink_moe_stack_decode(*common, self.status.data_ptr(), _abi.stream()))
        else:
            _abi.check(_abi.lib().ink_moe_stack_decode_tp(*common, self.rank, self.world, self.peer_regions,
                                                          self.status.data_ptr(), _abi.stream()))

    def check_status(self) -> None:
        """Host read (synchronises): raises if a bounded wait inside the kernel gave up, after
        putting the scratch back into its initial state so that the next launch is sound.

        With several ranks this is a COLLECTIVE: every rank must call it at the same point. The
        ranks agree on whether anyone failed (an abandoned launch on one rank leaves every rank's
        launch counts and tags out of step), and if so all of them zero scratch and symmetric
        region between two barriers, so that nobody stores into a region that is being cleared."""
        flags = self.status.clone()
        if self.world > 1:
            # (NCCL has no bitwise OR: the two bits are reduced apart, each with MAX)
            bits = torch.stack([flags & 1, (flags >> 1) & 1]).to(torch.int32)
            torch.distributed.all_reduce(bits, op=torch.distributed.ReduceOp.MAX, group=self.group)
            flags = bits[0] | (bits[1] << 1)
        flags = int(flags.item())
        self.status.zero_()
        if flags & 2:
            if self.world > 1:
                torch.cuda.synchronize()
                torch.distributed.barrier(self.group)   # no launch of any rank is still storing
            self.scratch.zero_()   # counters, launch count and tagged words start over
            if self.symmetric is not None:
                self.symmetric.zero_()
            if self.world > 1:
                torch.cuda.synchronize()
                torch.distributed.barrier(self.group)   # every region is clean before anyone launches again
            raise RuntimeError("moe_stack: a bounded wait inside the kernel timed out; the output is invalid")

    def seed_launch_count(self, launches: int) -> None:
        """Test hook: make the scratch look as if `launches` launches had already run (launch
        count and the two grid-wide counters of every block, which grow by one per thread block
        and launch), so that the wrap of the 32-bit counts can be reached without running
        2^32 / 148 launches first. CUDA-core variant on one GPU only; synchronises."""
        assert self.bank_maps is None and self.world == 1
        blocks = torch.cuda.get_device_properties(self.scratch.device).multi_processor_count
        words = self.scratch.view(torch.int32)
        sync_words = 8 * self.n_layers                       # [n_layers][8] counters at the start of the scratch
        epoch_at = (sync_words * 4 + 255) // 256 * 256 // 4  # the launch count follows, 256-byte aligned

        def as_i32(v: int) -> int:
            v &= 0xFFFFFFFF
            return v - (1 << 32) if v >= 1 << 31 else v

        torch.cuda.synchronize()
        words[:sync_words].view(self.n_layers, 8)[:, 0:2] = as_i32(launches * blocks)
        words[epoch_at] = as_i32(launches)
        torch.cuda.synchronize()

    TRACE_SLOTS = ("layer_start", "router_rows_done", "shared_gate_up_done", "routed_gate_up_done",
                   "shared_gate_up_everywhere", "shared_down_done", "routed_gate_up_everywhere", "activations_staged",
                   "routed_down_done", "down_everywhere", "norm_done", "x_digits_written", "producer_waits_for_routing",
                   "producer_has_routing", "producer_layer_issued", "x_digits_visible", "mma_gate_up_start", "mma_gate_up_end",
                   "mma_down_start", "mma_down_end", "scales_gate_up_end", "scales_down_end", "rows_sent", "norm_reduced",
                   "cycles_waited_router", "cycles_waited_shared_gate_up", "cycles_waited_routed_gate_up",
                   "cycles_waited_shared_down", "cycles_waited_routed_down", "cycles_producer_waited_for_slot", "cycles_busy_shared_gate_up", "cycles_busy_routed_gate_up")

    def trace(self) -> torch.Tensor:
        """Phase stamps of the last decode run with INKLING_STACK_TRACE=1: int64
        [n_layers, 256, 32]: nanosecond stamps in slots 0..23 (zero where a block did not stamp), SM clock
        cycles spent waiting or holding tiles in slots 24..31 (see TRACE_SLOTS). Synchronises."""
        offset = _abi.lib().ink_moe_stack_trace_offset(self.n_layers, self.hidden, self.intermediate, self.experts,
                                                       self.n_shared, self.top_k)
        raw = self.scratch[offset:offset + self.n_layers * 256 * 32 * 8].clone()
        return raw.view(torch.int64).view(self.n_layers, 256, 32).cpu()
