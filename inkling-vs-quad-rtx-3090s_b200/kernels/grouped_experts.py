"""Weight-bank naming shared by the decode and grouped paths."""
from __future__ import annotations


def expert_bank_names(quantized: bool) -> list[str]:
    """One expert's weight banks in pointer-table order (reference:
    kernels/grouped_experts.py:9-22): gate/up first, then down, each followed by its
    NVFP4 scale banks when quantized. The length is the pointer-table stride."""
    suffixes = ("", "_scale", "_scale2") if quantized else ("",)
    return [projection + suffix for projection in ("gate_up_proj", "down_proj") for suffix in suffixes]
