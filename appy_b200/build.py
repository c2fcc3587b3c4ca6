"""Build libappy_sm100.so in-tree with nvcc for sm_100a.

Usage: ``python -m appy_b200.build [--force] [--verbose]``.  The library is written
next to this file as ``appy_b200/libappy_sm100.so``; it links the CUDA runtime
statically and NVRTC dynamically, and does not need the CUDA driver library at load
time, so it can be loaded (not run) on a machine without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libappy_sm100.so")
STAMP = os.path.join(HERE, "libappy_sm100.stamp")

SOURCES = ["appy_shim.cu", "appy_prebuilt.cu", "appy_noalloc.cu"]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build libappy_sm100.so")
    return nvcc


def _sources() -> list[str]:
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _digest() -> str:
    h = hashlib.sha256()
    files = _sources() + [os.path.join(HERE, "..", "include", "appy_sm100.h")]
    tdir = os.path.join(CSRC, "templates")
    files += sorted(os.path.join(tdir, f) for f in os.listdir(tdir))
    for f in files:
        with open(f, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if sources changed since the last build; return its path."""
    digest = _digest()
    if not force and os.path.exists(LIB) and os.path.exists(STAMP):
        with open(STAMP) as fh:
            if fh.read().strip() == digest:
                return LIB
    cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
    cmd = [
        _nvcc(), "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-Xptxas", "-v" if verbose else "-O3",
        "-o", LIB, *_sources(),
        "-L" + os.path.join(cuda_home, "lib64"), "-lnvrtc",
        "-Xlinker", "-rpath," + os.path.join(cuda_home, "lib64"),
    ]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    with open(STAMP, "w") as fh:
        fh.write(digest)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
