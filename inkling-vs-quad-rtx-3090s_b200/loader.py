"""Resident placement of the routed experts' banks: the loader's side of the path.

The reference reads its per-rank pack into `{experts module: {global expert id: {bank: tensor}}}`
with records named `"<experts module>.<bank>/<expert id>"` and keeps only a few experts on the GPU
(utils/flashpack_cache.py:102-159, placement.json). Here every expert is resident, and the banks
of one kind of a layer go into ONE device allocation each, expert after expert: that is what lets
the tensor-core kernels address a layer's banks through four TMA descriptors
(`ResidentExperts.bank_layout`), and it is the order a sequential reader delivers them in anyway.
"""
from __future__ import annotations

from collections import defaultdict
from typing import Iterable, Mapping

import torch


def split_record_name(name: str) -> tuple[str, str, int]:
    """`"<experts module>.<bank>/<expert id>"` -> (module, bank, expert id), the reference's record
    naming (scripts/make_flashpack.py:97-100, utils/flashpack_cache.py:153-156)."""
    stem, _, expert = name.rpartition("/")
    module, _, bank = stem.rpartition(".")
    return module, bank, int(expert)


def pack_resident_experts(records: Mapping[str, torch.Tensor] | Iterable[tuple[str, torch.Tensor]], device,
                          ) -> dict[str, dict[int, dict[str, torch.Tensor]]]:
    """All records of this rank's pack -> the `expert_state_dict` that `apply_resident_plan` /
    `apply_fused_moe_plan` take, with every (module, bank) in one contiguous allocation on `device`
    and the per-expert tensors views into it. Expert ids of a module must be consecutive; a scalar
    bank (`*_scale2`) becomes a one-element FP32 view. Host tensors are copied one expert at a time
    (pinned source memory makes the copies asynchronous)."""
    items = records.items() if isinstance(records, Mapping) else records
    grouped: dict[tuple[str, str], dict[int, torch.Tensor]] = defaultdict(dict)
    for name, tensor in items:
        module, bank, expert = split_record_name(name)
        grouped[(module, bank)][expert] = tensor
    state: dict[str, dict[int, dict[str, torch.Tensor]]] = {}
    for (module, bank), by_expert in grouped.items():
        ids = sorted(by_expert)
        if ids != list(range(ids[0], ids[0] + len(ids))):
            raise ValueError(f"{module}.{bank}: expert ids are not consecutive")
        first = by_expert[ids[0]]
        shape = tuple(first.shape) if first.dim() else (1,)
        dtype = torch.float32 if bank.endswith("scale2") else first.dtype
        if dtype in (torch.float8_e4m3fn,):
            dtype = torch.uint8   # block scales travel as bytes
        block = torch.empty((len(ids), *shape), dtype=dtype, device=device)
        for slot, expert in enumerate(ids):
            source = by_expert[expert]
            if source.dtype == torch.float8_e4m3fn:
                source = source.view(torch.uint8)
            block[slot].copy_(source.reshape(shape).to(dtype), non_blocking=True)
            state.setdefault(module, {}).setdefault(expert, {})[bank] = block[slot]
    return state
