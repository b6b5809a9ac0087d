"""Builds libpeerkv.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m peerkv_b200.build [--force]

The shared object lands next to this file so it travels with the source tree;
nothing is cached outside the repository.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libpeerkv.so")
SOURCES = ["api.cu"]
HEADERS = ["ptx.cuh", "decode_kernel.cuh", "merge_kernel.cuh", "layer_kernels.cuh", "prefill_kernel.cuh", os.path.join("..", "..", "include", "peerkv.h")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _source_hash() -> str:
    import hashlib
    h = hashlib.sha256()
    for f in SOURCES + HEADERS:
        path = os.path.join(CSRC, f)
        h.update(f.encode())
        if os.path.exists(path):
            with open(path, "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


STAMP = LIB + ".srchash"


def _stale() -> bool:
    """The library is rebuilt unless it was built from exactly these sources (a content
    hash kept beside it; file times do not survive a copy of the tree)."""
    if not os.path.exists(LIB) or not os.path.exists(STAMP):
        return True
    with open(STAMP) as f:
        return f.read().strip() != _source_hash()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile if the library is missing or was built from other sources; returns its path."""
    if not force and not _stale():
        return LIB
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-Xptxas", "-v" if verbose else "-O3", "-shared", "-Xcompiler", "-fPIC",
           "-o", LIB + ".tmp"] + [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    os.replace(LIB + ".tmp", LIB)          # never a half-written library in the tree
    with open(STAMP, "w") as f:
        f.write(_source_hash() + "\n")
    if verbose:
        print(res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
