"""Builds oracle/_ref/: the reference's kernels/routed_decode.cu compiled for the CPU
behind oracle/ref_cpu_shim.h, one shared library per (K, QUANT). The sources are read
where they lie (nothing is copied); outputs go to oracle/_ref/ only. Test
infrastructure: used to generate tests/golden/ fixtures.

    python oracle/build_ref.py <reference_root>      (or INKLING_REFERENCE_ROOT=<reference_root>)
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
WIDTHS = (32, 64, 128, 256, 512, 1024, 2048, 4096)


def lib_path(k: int, quant: int) -> Path:
    return OUT / f"ref_routed_decode_K{k}_Q{quant}.so"


def reference_root(explicit: str | None = None) -> Path | None:
    """The reference checkout: the argument, else the environment variable
    INKLING_REFERENCE_ROOT, else a directory named `reference` beside this repository."""
    for candidate in (explicit, os.environ.get("INKLING_REFERENCE_ROOT"), HERE.parents[1] / "reference"):
        if candidate and (Path(candidate) / "kernels" / "routed_decode.cu").exists():
            return Path(candidate)
    return None


def build(root: str | None = None) -> list[Path]:
    """NVFP4 (QUANT=1) and BF16 (QUANT=0) builds of every width; no-op without a checkout."""
    root = reference_root(root)
    if root is None:
        return []
    source = root / "kernels" / "routed_decode.cu"
    OUT.mkdir(exist_ok=True)
    built = []
    for quant in (1, 0):
        for k in WIDTHS:
            target = lib_path(k, quant)
            if not target.exists() or target.stat().st_mtime < source.stat().st_mtime:
                subprocess.run(
                    ["g++", "-std=c++20", "-O1", "-shared", "-fPIC", "-pthread", "-x", "c++",
                     f"-DK={k}", f"-DQUANT={quant}", f'-DREF_CU="{source}"', "-I", str(HERE),
                     str(HERE / "ref_routed_decode_driver.cpp"), "-o", str(target)],
                    check=True)
            built.append(target)
    return built


if __name__ == "__main__":
    for path in build(*sys.argv[1:2]):
        print(path)
