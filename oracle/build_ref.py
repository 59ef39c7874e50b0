"""Builds oracle/_ref/: the reference's kernels/routed_decode.cu compiled for the CPU
behind oracle/ref_cpu_shim.h, one shared library per (K, QUANT). The sources are read
where they lie (nothing is copied); outputs go to oracle/_ref/ only. Test
infrastructure: used to generate tests/golden/ fixtures.

    python oracle/build_ref.py [reference_root]
"""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
WIDTHS = (32, 64, 128, 256, 512, 1024, 2048, 4096)


def lib_path(k: int, quant: int) -> Path:
    return OUT / f"ref_routed_decode_K{k}_Q{quant}.so"


def build(reference_root: str = "/root/reference") -> list[Path]:
    source = Path(reference_root) / "kernels" / "routed_decode.cu"
    if not source.exists():
        return []
    OUT.mkdir(exist_ok=True)
    built = []
    for k in WIDTHS:
        target = lib_path(k, 1)
        if not target.exists() or target.stat().st_mtime < source.stat().st_mtime:
            subprocess.run(
                ["g++", "-std=c++20", "-O1", "-shared", "-fPIC", "-pthread", "-x", "c++",
                 f"-DK={k}", "-DQUANT=1", f'-DREF_CU="{source}"', "-I", str(HERE),
                 str(HERE / "ref_routed_decode_driver.cpp"), "-o", str(target)],
                check=True)
        built.append(target)
    return built


if __name__ == "__main__":
    for path in build(*sys.argv[1:2]):
        print(path)
