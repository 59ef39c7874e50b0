"""Ahead-of-time build of the CUDA library for sm_100a.

    python build.py            # writes ../libinkling_b200.so

The shared object exports the C ABI declared in include/inkling_b200.h. It is built
in-tree (next to the Python package) and loaded with ctypes; nothing is JIT-compiled
at run time.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PACKAGE = CSRC.parent
LIBRARY = PACKAGE / "libinkling_b200.so"
SOURCES = ("router_plan.cu", "routed_decode.cu", "stream_decode.cu", "moe_stack.cu", "grouped_experts.cu", "grouped_tc.cu", "glue.cu", "attention.cu")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas=-v",
]


def nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if candidate and (os.path.sep not in candidate or os.path.exists(candidate)):
            return candidate
    raise RuntimeError("nvcc not found")


def needs_build() -> bool:
    if not LIBRARY.exists():
        return True
    stamp = LIBRARY.stat().st_mtime
    inputs = [CSRC / s for s in SOURCES] + list(CSRC.glob("*.cuh")) + [Path(__file__)] + [PACKAGE.parent / "include" / "inkling_b200.h"]
    return any(p.stat().st_mtime > stamp for p in inputs)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIBRARY
    objects = []
    build_dir = CSRC / "build"
    build_dir.mkdir(exist_ok=True)
    for source in SOURCES:
        obj = build_dir / (Path(source).stem + ".o")
        cmd = [nvcc(), *NVCC_FLAGS, "-c", str(CSRC / source), "-o", str(obj)]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or result.returncode:
            sys.stderr.write(result.stdout + result.stderr)
        if result.returncode:
            raise RuntimeError(f"nvcc failed on {source}")
        objects.append(str(obj))
    cmd = [nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", *objects, "-o", str(LIBRARY)]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode:
        sys.stderr.write(result.stdout + result.stderr)
        raise RuntimeError("link failed")
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
