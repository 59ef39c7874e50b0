"""Expert routing plan for a placement in which every expert is resident in HBM.

Keeps the launch syntax of the reference's Triton kernels
(kernels/expert_planner.py:11-33 `expert_plan[grid](...)`, :117-125
`expert_copy[grid](...)`) so that the host code that calls them reads the same.
"""
from __future__ import annotations

from . import _abi


class _Launcher:
    """`kernel[grid](*args)` in the manner of a Triton kernel; the grid is accepted for
    source compatibility and ignored (the library sizes its own launches)."""

    def __init__(self, fn):
        self._fn = fn
        self.__doc__ = fn.__doc__

    def __getitem__(self, grid):
        return self._fn


def _expert_plan(Indices, Sources, Resident, Destinations, SlotExperts, Ages, Clock, CopyExperts, Pointers,
                 Experts, Counts, Rows, START, LOCAL, SLOTS, STRIDE, ROUTES, CAPACITY, E=None, S=None, R=None,
                 num_warps=None):
    """Groups token routing by expert and writes the pointer table.

    Arguments as the reference's expert_plan. With every expert resident there is no
    slot cache: SLOTS must be 0 and Resident/Destinations/SlotExperts/Ages/CopyExperts
    are not touched; Clock is not advanced. E, S, R and num_warps (Triton tuning
    constants) are ignored.
    """
    if SLOTS != 0:
        raise RuntimeError("expert_plan: this build keeps every expert resident (SLOTS must be 0); "
                           "the LRU slot cache of the reference is not built")
    _abi.require_cuda(Indices, Sources, Pointers, Experts, Counts, Rows)
    assert Indices.is_contiguous() and Sources.is_contiguous() and Rows.is_contiguous()
    _abi.check(_abi.lib().ink_expert_plan(
        Indices.data_ptr(), Sources.data_ptr(), Pointers.data_ptr(), Experts.data_ptr(), Counts.data_ptr(),
        Rows.data_ptr(), START, LOCAL, STRIDE, ROUTES, CAPACITY, _abi.stream()))


def _expert_copy(Sources, Destinations, CopyExperts, SIZES, STRIDE, BLOCK, WORKERS):
    """No cache slots exist under the resident placement, so there is nothing to copy."""
    if CopyExperts.numel() != 0:
        raise RuntimeError("expert_copy: no slot cache in this build (every expert is resident)")


expert_plan = _Launcher(_expert_plan)
expert_copy = _Launcher(_expert_copy)
