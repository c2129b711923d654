"""Builds libprichs_moe.so (the C-ABI library) in-tree with nvcc for sm_100a.

Usage: python -m prichs_b200.build [--force] [--verbose] [--check]
The shared object lands next to the sources' package (prichs_b200/libprichs_moe.so) so that it travels with
the tree; nothing is installed into site-packages.
"""
from __future__ import annotations

import os
import subprocess
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_PKG, "csrc")
LIB_PATH = os.path.join(_PKG, "libprichs_moe.so")
CHECK_LIB_PATH = os.path.join(_PKG, "libprichs_moe_check.so")  # same sources with -DPRICHS_BOUNDS_CHECK
SOURCES = ["prichs_moe.cu"]
HEADERS = sorted(f for f in os.listdir(_CSRC) if f.endswith(".cuh")) + ["../../include/prichs_moe.h"]

NVCC_FLAGS = [
    "-ldl",
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def needs_build(path: str = LIB_PATH) -> bool:
    if not os.path.exists(path):
        return True
    t = os.path.getmtime(path)
    deps = [os.path.join(_CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(p) > t for p in deps)


def build(force: bool = False, verbose: bool = False, check: bool = False) -> str:
    """Builds the library (check=True: the index-checking build, libprichs_moe_check.so) unless it is up to date."""
    path = CHECK_LIB_PATH if check else LIB_PATH
    if not force and not needs_build(path):
        return path
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + (["-DPRICHS_BOUNDS_CHECK"] if check else [])
    cmd += [os.path.join(_CSRC, s) for s in SOURCES] + ["-o", path]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed building {os.path.basename(path)}")
    return path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, check="--check" in sys.argv))
