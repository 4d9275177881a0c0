"""Builds the C-ABI shared library (hand-written CUDA for sm_100a) in-tree with nvcc.

    python -m kv_cache_b200.build            # build if sources are newer than the library
    python -m kv_cache_b200.build --force

The library lands in kv_cache_b200/_lib/libkvcache_b200.so; nothing is installed elsewhere.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "_lib"
LIB_PATH = LIB_DIR / "libkvcache_b200.so"
UNITY = CSRC / "kvcache_b200.cu"

NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-shared",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    # IEEE division / sqrt and no flush-to-zero: codes and scales must match the CPU oracle bit for bit.
    "-prec-div=true", "-prec-sqrt=true", "-ftz=false",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; the CUDA library cannot be built")


def sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "kvcache_b200.h"])


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(s.stat().st_mtime > built for s in sources())


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not is_stale():
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    extra = os.environ.get("KVB_NVCC_EXTRA", "").split()       # e.g. -D switches for experiments
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-o", str(LIB_PATH), str(UNITY)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed ({res.returncode}):\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
