"""Builds the C-ABI shared library (hand-written CUDA for sm_100a) in-tree with nvcc.

    python -m kv_cache_b200.build            # build if sources are newer than the library
    python -m kv_cache_b200.build --force

The library lands in kv_cache_b200/_lib/libkvcache_b200.so; nothing is installed elsewhere.
"""
from __future__ import annotations

import fcntl
import hashlib
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


STAMP_PATH = LIB_DIR / "libkvcache_b200.srchash"


def source_hash() -> str:
    """Hash of every source the library is built from (content, not modification times: a copy of the tree
    to another machine must not look stale)."""
    h = hashlib.sha256()
    for s in sources():
        h.update(s.name.encode())
        h.update(s.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_stale() -> bool:
    if not LIB_PATH.exists() or not STAMP_PATH.exists():
        return True
    return STAMP_PATH.read_text().strip() != source_hash()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the library when its sources changed. Safe when several processes (the ranks of one node) call
    it at once: one holds a file lock and builds into a temporary file that is renamed into place, the others
    wait for the lock and find the library fresh."""
    if not force and not is_stale():
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    with open(LIB_DIR / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not is_stale():
                return LIB_PATH
            digest = source_hash()
            tmp = LIB_DIR / f".libkvcache_b200.{os.getpid()}.so.tmp"
            cmd = [_nvcc(), *NVCC_FLAGS, "-o", str(tmp), str(UNITY)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
                print(" ".join(cmd), flush=True)
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                tmp.unlink(missing_ok=True)
                raise RuntimeError(f"nvcc failed ({res.returncode}):\n{res.stdout}\n{res.stderr}")
            if verbose:
                print(res.stderr)
            os.replace(tmp, LIB_PATH)
            STAMP_PATH.write_text(digest + "\n")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
