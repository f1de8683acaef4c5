"""Generate golden vectors from the reference's own torch path.

Runs ONLY where a Mooncake checkout is available (argument `--reference`, or
the environment variable `MOONCAKE_SRC`). It loads
`mooncake-wheel/mooncake/mooncake_ep_buffer.py` by file path, builds the
`Buffer` object without its native runtime, and calls the reference's
`_fallback_dispatch` / `_fallback_combine` on CPU tensors with a gloo group
(gloo stands in for the reference's own `mooncake-cpu` backend; one shim:
gloo wants the output of `all_gather_into_tensor` flat, the reference passes
`[R, T, ...]`).

The vectors land in `tests/golden/*.pt`; tests read only those files.

    python tests/golden/make_golden.py --reference <path to the Mooncake tree>
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.util
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))

# name -> config. `tokens` is per rank (uneven on purpose in some cases).
CASES = {
    # the CPU-runnable case: 2 ranks, 128 tokens, hidden 2048, 16 experts, top-4
    "c1_bf16": dict(R=2, tokens=[128, 128], M=128, H=2048, E=16, K=4, fp8=False,
                    routing="softmax_topk", mask=0, full=False, seed=0),
    "c1_fp8": dict(R=2, tokens=[128, 128], M=128, H=2048, E=16, K=4, fp8=True,
                   routing="softmax_topk", mask=0, full=False, seed=0),
    # small, fully stored
    "small_fp8_uneven": dict(R=2, tokens=[16, 13], M=16, H=256, E=8, K=3, fp8=True,
                             routing="uniform", mask=5, full=True, seed=11),
    "small_bf16_uneven": dict(R=2, tokens=[9, 16], M=16, H=256, E=8, K=3, fp8=False,
                              routing="uniform", mask=4, full=True, seed=12),
    "single_rank_fp8": dict(R=1, tokens=[8], M=8, H=128, E=4, K=2, fp8=True,
                            routing="uniform", mask=2, full=True, seed=13),
    "empty_rank_bf16": dict(R=2, tokens=[0, 6], M=8, H=128, E=4, K=2, fp8=False,
                            routing="uniform", mask=0, full=True, seed=14),
}


def make_inputs(cfg: dict, rank: int):
    """Seeded inputs of one rank; `tests/` regenerates them with this function."""
    g = torch.Generator().manual_seed(cfg["seed"] * 1000 + rank)
    T, H, E, K = cfg["tokens"][rank], cfg["H"], cfg["E"], cfg["K"]
    x = torch.randn((T, H), generator=g, dtype=torch.float32).to(torch.bfloat16)
    logits = torch.randn((T, E), generator=g, dtype=torch.float32)
    if cfg["routing"] == "softmax_topk":
        p = torch.softmax(logits, dim=-1)
        w, idx = torch.topk(p, K, dim=-1)
        w = (w / w.sum(dim=-1, keepdim=True)).to(torch.float32)
    else:
        idx = torch.topk(logits, K, dim=-1)[1]
        w = torch.softmax(torch.rand((T, K), generator=g, dtype=torch.float32), dim=-1)
    idx = idx.to(torch.int64).contiguous()
    for _ in range(cfg["mask"] if T else 0):
        t = int(torch.randint(0, T, (1,), generator=g))
        k = int(torch.randint(0, K, (1,), generator=g))
        idx[t, k] = -1
    return x.contiguous(), idx, w.contiguous()


def expert_op(recv_bf16: torch.Tensor, rank: int, L: int) -> torch.Tensor:
    """Mock expert of the CPU-runnable case: y = x * (1 + e/16), fp32 then bf16."""
    out = torch.empty_like(recv_bf16)
    for le in range(L):
        e = rank * L + le
        out[le] = (recv_bf16[le].float() * (1.0 + e / 16.0)).to(torch.bfloat16)
    return out


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def _load_reference(reference_root: str):
    path = os.path.join(reference_root, "mooncake-wheel", "mooncake", "mooncake_ep_buffer.py")
    spec = importlib.util.spec_from_file_location("ref_mooncake_ep_buffer", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _worker(rank: int, name: str, cfg: dict, reference_root: str, port: int, out_dir: str):
    R = cfg["R"]
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=R)
    ref = _load_reference(reference_root)

    orig = dist.all_gather_into_tensor

    def flat_all_gather_into_tensor(out, inp, group=None, **kw):
        return orig(out.view(-1, *inp.shape[1:]), inp, group=group, **kw)

    dist.all_gather_into_tensor = flat_all_gather_into_tensor

    buf = ref.Buffer.__new__(ref.Buffer)
    buf.rank, buf.group_size, buf.group, buf.backend = rank, R, dist.group.WORLD, dist.group.WORLD
    buf._use_fallback = True
    buf._fallback_next_combine_buffer = None
    buf._warned_active_ranks_without_mooncake_backend = True

    x, idx, w = make_inputs(cfg, rank)
    M, E, H = cfg["M"], cfg["E"], cfg["H"]
    L = E // R
    recv_x, scales, recv_count, src_info, layout_range, _, _ = buf._fallback_dispatch(
        x, idx, M, E, cfg["fp8"], False)
    if cfg["fp8"]:
        deq = (recv_x.to(torch.float32).view(L, R * M, -1, 128)
               * scales.view(L, R * M, -1, 1)).view(L, R * M, H).to(torch.bfloat16)
    else:
        deq = recv_x
    y = expert_op(deq, rank, L)
    out = torch.empty((x.size(0), H), dtype=torch.bfloat16)
    combined, _, _ = buf._fallback_combine(y, idx, w, src_info, layout_range, M, E,
                                           False, False, out)
    rec = dict(cfg=cfg, rank=rank,
               in_sha=dict(x=sha(x), idx=sha(idx), w=sha(w)),
               recv_count=recv_count.clone(), src_info=src_info.clone(),
               layout_range=layout_range.clone())
    # valid rows only, per expert
    rx_u8 = recv_x.view(torch.uint8) if cfg["fp8"] else recv_x
    rec["recv_x_sha"] = [sha(rx_u8[le, :int(recv_count[le])]) for le in range(L)]
    if cfg["fp8"]:
        rec["scales_sha"] = [sha(scales[le, :int(recv_count[le])]) for le in range(L)]
    rec["combined_sha"] = sha(combined)
    if cfg["full"]:
        rec["recv_x"] = rx_u8.clone()
        rec["scales"] = scales.clone() if cfg["fp8"] else None
        rec["y"] = y.clone()
        rec["combined"] = combined.clone()
    else:
        # a thin, fully stored slice so a mismatch can be localised
        rec["recv_x_head"] = [rx_u8[le, :min(4, int(recv_count[le]))].clone() for le in range(L)]
        if cfg["fp8"]:
            rec["scales_head"] = [scales[le, :min(4, int(recv_count[le]))].clone() for le in range(L)]
        rec["combined_head"] = combined[:8].clone()
    torch.save(rec, os.path.join(out_dir, f"{name}.rank{rank}.part"))
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("MOONCAKE_SRC"),
                    required="MOONCAKE_SRC" not in os.environ,
                    help="root of the Mooncake source tree (or set MOONCAKE_SRC)")
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    torch.set_num_threads(2)
    port = 29610
    for name, cfg in CASES.items():
        if args.only and name != args.only:
            continue
        port += 1
        mp.spawn(_worker, args=(name, cfg, args.reference, port, HERE), nprocs=cfg["R"], join=True)
        parts = []
        for r in range(cfg["R"]):
            p = os.path.join(HERE, f"{name}.rank{r}.part")
            parts.append(torch.load(p))
            os.remove(p)
        torch.save(dict(name=name, torch=torch.__version__, ranks=parts),
                   os.path.join(HERE, f"{name}.pt"))
        print(name, [int(p["recv_count"].sum()) for p in parts], flush=True)


if __name__ == "__main__":
    sys.exit(main())
