"""Builds libmcep.so (the CUDA kernels and the C ABI) in-tree with nvcc, for sm_100a only."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
# MCEP_LIB points the package at a library built elsewhere (e.g. a diagnostic build)
LIB = os.environ.get("MCEP_LIB") or os.path.join(HERE, "libmcep.so")
SOURCES = ["ep_kernels.cu", "ep_runtime.cu", "ep_noalloc.cu"]
HEADERS = ["ep_kernels.cuh", "ep_device.cuh", os.path.join("..", "..", "include", "mcep.h")]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("mooncake_b200: nvcc not found; cannot build libmcep.so")
    cmd = [nvcc, "-std=c++17", "-O3", "-lineinfo",
           "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xcompiler", "-fPIC", "-shared", "-cudart", "static",
           "-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    cmd[1:1] = os.environ.get("MCEP_NVCC_FLAGS", "").split()  # e.g. -DMCEP_PHASE_TRACE
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
