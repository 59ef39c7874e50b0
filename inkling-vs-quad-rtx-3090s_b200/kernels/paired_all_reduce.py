"""All-reduce of a rank's partial layer output.

The reference's kernels/paired_all_reduce.py:146-160 exists because its four GPUs sit
in two NVLink pairs joined by PCIe. On an NVSwitch box every peer is one hop away, so
the sum is one NCCL all-reduce (captured in the decode graph like any other launch).
Same signature and return convention: the reduced tensor is returned.
"""
from __future__ import annotations

import torch.distributed as dist


def all_reduce(x, group=None):
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(x, group=group)
    return x
