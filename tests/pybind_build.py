"""Compiles the pybind11 binding of the C ABI (mooncake_b200/csrc/ep_py_mcep.cpp)
into a directory and imports it. Used by the CPU surface test and the GPU test."""
from __future__ import annotations

import importlib.util
import os
import subprocess
import sys
import sysconfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build_and_import(out_dir: str):
    import pybind11
    from mooncake_b200 import build as lib_build
    lib = lib_build.build()
    lib_dir = os.path.dirname(lib)
    out = os.path.join(out_dir, "_ep" + sysconfig.get_config_var("EXT_SUFFIX"))
    cmd = ["g++", "-O1", "-shared", "-fPIC", "-std=c++17",
           "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
           "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "mooncake_b200", "csrc", "ep_py_mcep.cpp"), "-o", out,
           "-L", lib_dir, "-l:" + os.path.basename(lib), "-Wl,-rpath," + lib_dir]
    subprocess.run(cmd, check=True)
    spec = importlib.util.spec_from_file_location("_ep", out)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
