"""Builds libmcep.so (the CUDA kernels and the C ABI) in-tree with nvcc, for sm_100a only."""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
# MCEP_LIB points the package at a library built elsewhere (e.g. a diagnostic build)
LIB = os.environ.get("MCEP_LIB") or os.path.join(HERE, "libmcep.so")
SOURCES = ["ep_kernels.cu", "ep_runtime.cu", "ep_noalloc.cu", "ep_elastic_kernels.cu",
           "ep_elastic.cu"]
HEADERS = ["ep_kernels.cuh", "ep_device.cuh", "ep_elastic.cuh", "ep_runtime_internal.h",
           os.path.join("..", "..", "include", "mcep.h")]


STAMP = LIB + ".sources"  # digest of the sources the library was built from


def _digest() -> str:
    h = hashlib.sha256()
    h.update(os.environ.get("MCEP_NVCC_FLAGS", "").encode())
    for f in SOURCES + HEADERS:
        path = os.path.join(CSRC, f)
        if os.path.exists(path):
            with open(path, "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


def _stale() -> bool:
    """True when the library is missing or was built from other sources (file
    contents are compared, not times: a copy of the tree keeps no times)."""
    if not os.path.exists(LIB):
        return True
    try:
        with open(STAMP) as fh:
            return fh.read().strip() != _digest()
    except OSError:
        return True


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    # several processes of one job may import the package at once: one builds
    with open(LIB + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not _stale():
                return LIB
            return _build_locked(force, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(force: bool, verbose: bool) -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        if os.path.exists(LIB) and not force:
            return LIB  # a prebuilt library and no compiler: use what is there
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
    with open(STAMP, "w") as fh:
        fh.write(_digest())
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
