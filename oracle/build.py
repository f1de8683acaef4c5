"""Build recipes for the CPU oracle (test infrastructure, never shipped).

`build_oracle()` compiles `ep_oracle.c` (the plain-C restatement of the
reference arithmetic) into `oracle/libep_oracle.so` with gcc.

`build_reference_kernels()` compiles the reference's own CUDA translation unit
`mooncake-ep/src/mooncake_ep_kernel.cu`, from where it lies in a Mooncake
checkout, together with the small host harness `ref_harness.cu` of this
directory into `oracle/_ref/libmooncake_ep_ref.so`. Only build products go to
`oracle/_ref/`; no reference source is copied. The two rdma-core headers the
translation unit includes are not installed on the build machine, so
declaration-only stand-ins are generated into `oracle/_ref/stub/` (the RDMA
branch they serve is never taken when the queue-pair tables are null).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libep_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libmooncake_ep_ref.so")


def _newer(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "ep_oracle.c")
    if not force and _newer(ORACLE_SO, src):
        return ORACLE_SO
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        raise RuntimeError("oracle: no C compiler found (gcc/cc)")
    cmd = [cc, "-O2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC",
           "-o", ORACLE_SO, src, "-lm"]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


_VERBS_STUB = """\
// Declaration-only stand-in for <infiniband/verbs.h>: the EP kernel
// translation unit needs the names to parse, never the behaviour.
#pragma once
#include <stdint.h>
struct ibv_context; struct ibv_pd; struct ibv_mr; struct ibv_cq; struct ibv_qp;
struct ibv_device; struct ibv_srq; struct ibv_comp_channel;
enum ibv_mtu { IBV_MTU_256 = 1, IBV_MTU_512 = 2, IBV_MTU_1024 = 3,
               IBV_MTU_2048 = 4, IBV_MTU_4096 = 5 };
enum ibv_port_state { IBV_PORT_NOP = 0, IBV_PORT_DOWN = 1, IBV_PORT_INIT = 2,
                      IBV_PORT_ARMED = 3, IBV_PORT_ACTIVE = 4 };
struct ibv_port_attr { enum ibv_port_state state; enum ibv_mtu max_mtu;
                       enum ibv_mtu active_mtu; int gid_tbl_len;
                       uint16_t lid; uint8_t link_layer; };
union ibv_gid { uint8_t raw[16];
                struct { uint64_t subnet_prefix; uint64_t interface_id; } global; };
"""

_MLX5_STUB = """\
// Declaration-only stand-in for <infiniband/mlx5dv.h> (see verbs.h stub).
#pragma once
#include <stdint.h>
#include <linux/types.h>
#include <infiniband/verbs.h>
struct mlx5_wqe_ctrl_seg { uint32_t opmod_idx_opcode; uint32_t qpn_ds;
                           uint8_t signature; uint8_t rsvd[2]; uint8_t fm_ce_se;
                           uint32_t imm; };
struct mlx5_wqe_raddr_seg { uint64_t raddr; uint32_t rkey; uint32_t reserved; };
struct mlx5_wqe_data_seg { uint32_t byte_count; uint32_t lkey; uint64_t addr; };
struct mlx5_wqe_atomic_seg { uint64_t swap_add; uint64_t compare; };
struct mlx5_wqe_inl_data_seg { uint32_t byte_count; };
struct mlx5_cqe64 { uint8_t rsvd0[40]; uint64_t timestamp; uint8_t rsvd1[12];
                    uint16_t wqe_counter; uint8_t signature; uint8_t op_own; };
struct mlx5dv_devx_obj; struct mlx5dv_devx_umem; struct mlx5dv_devx_uar;
enum { MLX5_WQE_CTRL_CQ_UPDATE = 2 << 2 };
enum { MLX5_OPCODE_RDMA_WRITE = 0x08, MLX5_OPCODE_ATOMIC_FA = 0x12,
       MLX5_OPCODE_ATOMIC_MASKED_FA = 0x15, MLX5_OPCODE_NOP = 0x00 };
enum { MLX5_INLINE_SEG = 0x80000000 };
"""


def find_mooncake_src() -> str | None:
    """Where the Mooncake sources lie: the environment variable MOONCAKE_SRC, or a
    checkout named `reference` beside this repository. None when there is none."""
    marker = os.path.join("mooncake-ep", "src", "mooncake_ep_kernel.cu")
    cands = [os.environ.get("MOONCAKE_SRC"),
             os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.exists(os.path.join(c, marker)):
            return c
    return None


def build_reference_kernels(reference_root: str | None = None,
                            force: bool = False) -> str | None:
    """Compile the reference kernel TU + harness. Returns the .so path, or
    None when no Mooncake checkout is present (then a prebuilt .so, if any,
    is used as is)."""
    reference_root = reference_root or find_mooncake_src()
    if reference_root is None:
        return REF_SO if os.path.exists(REF_SO) else None
    ref_cu = os.path.join(reference_root, "mooncake-ep", "src",
                          "mooncake_ep_kernel.cu")
    harness = os.path.join(HERE, "ref_harness.cu")
    if not os.path.exists(ref_cu) or not os.path.exists(harness):
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, ref_cu, harness):
        return REF_SO
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    stub = os.path.join(REF_DIR, "stub", "infiniband")
    os.makedirs(stub, exist_ok=True)
    with open(os.path.join(stub, "verbs.h"), "w") as f:
        f.write(_VERBS_STUB)
    with open(os.path.join(stub, "mlx5dv.h"), "w") as f:
        f.write(_MLX5_STUB)
    cmd = [nvcc, "-std=c++17", "-O3", "--expt-relaxed-constexpr", "-DUSE_CUDA",
           "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-I", os.path.join(REF_DIR, "stub"),
           "-I", os.path.join(reference_root, "mooncake-ep", "include"),
           "-I", os.path.join(reference_root, "mooncake-transfer-engine", "include"),
           "-shared", "-Xcompiler", "-fPIC", "-cudart", "static",
           "-o", REF_SO, ref_cu, harness]
    subprocess.run(cmd, check=True)
    return REF_SO


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    if "--ref" in sys.argv:
        print(build_reference_kernels(force="--force" in sys.argv))
