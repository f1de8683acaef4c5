#!/usr/bin/env python
"""EP dispatch + combine benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...      # the CPU restatement of the reference path

A step is one MoE layer's token exchange: `Buffer.dispatch` then `Buffer.combine`
on one batch of synthetic tokens per rank (the mock expert between them is not
timed, as in the reference's harness, mooncake-ep/benchmarks/ep_benchmark/
run_ep_benchmark.py:316-352). Default workload: the DeepSeek-V3-shaped decode
case (128 tokens per rank, hidden 7168, 256 experts, top-8, FP8 dispatch, bf16
combine) with the experts split evenly over the N ranks. Rank 0 prints one JSON
line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: tokens/rank, hidden, experts, top-k, fp8 dispatch, routing
    "c2": dict(T=128, H=7168, E=256, K=8, fp8=True, routing="uniform",
               desc="DeepSeek-V3-shaped decode: 128 tok/rank, hidden 7168, 256 experts, top-8, "
                    "FP8 e4m3 dispatch + fp32 scales, bf16 combine"),
    "c3": dict(T=4096, H=7168, E=256, K=8, fp8=False, routing="uniform",
               desc="DeepSeek-V3-shaped prefill: 4096 tok/rank, hidden 7168, 256 experts, top-8, "
                    "bf16 dispatch, bf16 combine"),
    "c4": dict(T=256, H=4096, E=128, K=8, fp8=True, routing="zipf1.2",
               desc="Qwen3-235B-shaped: 256 tok/rank, hidden 4096, 128 experts, top-8 Zipf(1.2), "
                    "FP8 dispatch, bf16 combine"),
    "c5": dict(T=128, H=4096, E=8, K=2, fp8=False, routing="uniform",
               desc="Mixtral-shaped: hidden 4096, 8 experts, top-2, bf16"),
}
L2_FLUSH_BYTES = 512 << 20  # > 126 MB of L2


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=None, help="override tokens per rank")
    ap.add_argument("--e2e-steps", type=int, default=30)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-flush", action="store_true",
                    help="diagnosis only: leave L2 warm between steps (numbers are not reportable)")
    ap.add_argument("--force-staged", action="store_true",
                    help="single rank: go through staging + flags like a multi-rank group")
    ap.add_argument("--inactive-rank", type=int, default=-1,
                    help="mark this rank inactive on every rank; it makes no call")
    return ap.parse_args()


def workload(args):
    w = dict(WORKLOADS[args.workload])
    if args.tokens is not None:
        w["T"] = args.tokens
    w["name"] = args.workload
    return w


def make_inputs(w, rank, seed=2026):
    import torch
    g = torch.Generator().manual_seed(seed + rank)  # per-rank seed, as the reference's harness
    T, H, E, K = w["T"], w["H"], w["E"], w["K"]
    x = torch.randn((T, H), generator=g).to(torch.bfloat16)
    if w["routing"] == "uniform":
        scores = torch.randn((T, E), generator=g)
    else:
        alpha = float(w["routing"][4:])
        logp = -alpha * torch.log(torch.arange(1, E + 1, dtype=torch.float32))
        logp = logp - torch.logsumexp(logp, dim=0)
        u = torch.rand((T, E), generator=g).clamp(min=1e-20)
        scores = logp.unsqueeze(0) - torch.log(-torch.log(u))
    idx = torch.topk(scores, K, dim=-1)[1].to(torch.int64).contiguous()
    wts = torch.softmax(torch.rand((T, K), generator=g), dim=-1).float().contiguous()
    return x, idx, wts


# ----------------------------------------------------------------------------------------
# algorithmic bytes (what the roofline fractions are computed from)
# ----------------------------------------------------------------------------------------
def algorithmic_bytes(w, R, sel):
    """Bytes one rank must move per launch of each kernel, from the workload alone."""
    T, H, K = w["T"], w["H"], w["K"]
    S = H // 128
    payload = (H + 4 * S) if w["fp8"] else 2 * H   # per (token, selected expert)
    msg = payload + 16                             # plus the 16-byte header the reference counts
    b = {}
    # single rank: x read once, packed outputs written once; combine gathers and writes once
    b["ep_dispatch_send_direct"] = T * 2 * H + sel * payload + 8 * T * K + 4 * sel
    b["ep_combine_reduce_direct"] = sel * 2 * H + T * 2 * H + 12 * T * K
    # staged (R > 1): every kernel reads its input once and writes its output once
    b["ep_dispatch_send"] = T * 2 * H + sel * msg
    b["ep_dispatch_recv"] = 2 * sel * payload
    b["ep_combine_send"] = 2 * sel * 2 * H
    b["ep_combine_reduce"] = sel * 2 * H + T * 2 * H
    # both phases of a call in one launch (small batches in a group)
    b["ep_dispatch"] = b["ep_dispatch_send"] + b["ep_dispatch_recv"]
    b["ep_combine"] = b["ep_combine_send"] + b["ep_combine_reduce"]
    return b


# ----------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=fd, stderr=subprocess.DEVNULL)
            os.close(fd)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [s.strip() for s in line.split(",")]
                if len(f) < 9:
                    continue
                sm.append(float(f[1])), mx.append(float(f[2]))
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                    "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if not sm:
            return None
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------------------
# CPU legs (the oracle port of the reference's torch path)
# ----------------------------------------------------------------------------------------
def cpu_layer_seconds(w, R, budget_s, warmup=1, steps=50):
    """Times dispatch+combine of all R ranks with the CPU restatement of the
    reference's torch path (same arithmetic: amax/448 scales, bf16 running sum):
    `warmup` untimed layers, then `steps` timed ones. The time budget can cut
    both short (at least one of each runs). Returns (seconds per layer, timed
    layers run, warm-up layers run)."""
    import torch
    from oracle import ep_oracle as ora
    T, H, E, K = w["T"], w["H"], w["E"], w["K"]
    ins = [make_inputs(w, r) for r in range(R)]
    xs, idxs, ws = [i[0] for i in ins], [i[1] for i in ins], [i[2] for i in ins]
    L = E // R

    def layer():
        t0 = time.perf_counter()
        res = ora.dispatch(xs, idxs, T, E, w["fp8"], arith="fallback")
        t1 = time.perf_counter()
        ys = []
        for r in range(R):  # mock expert, not timed
            if w["fp8"]:
                ys.append(ora.fp8_dequant(res[r]["recv_x"].view(-1, H),
                                          res[r]["scales"].view(-1, H // 128)).view(L, -1, H))
            else:
                ys.append(res[r]["recv_x"])
        t2 = time.perf_counter()
        ora.combine(ys, idxs, ws, res, T, E, arith="fallback")
        t3 = time.perf_counter()
        return (t1 - t0) + (t3 - t2)

    t_start = time.perf_counter()
    warm = 0
    while warm < max(1, warmup):
        layer()
        warm += 1
        if time.perf_counter() - t_start > budget_s / 4:
            break
    times = []
    while len(times) < max(1, steps):
        times.append(layer())
        if time.perf_counter() - t_start > budget_s:
            break
    return sum(times) / len(times), len(times), warm


def run_reference_arm(args):
    """`--impl reference`: the reference's CPU path (oracle port) on the host cores."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    w = workload(args)
    R = args.gpus
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sec, iters, warm = cpu_layer_seconds(w, R, budget_s=150.0, warmup=args.warmup, steps=args.steps)
    value = w["T"] * R / sec
    line = {
        "impl": "reference", "metric": "ep_dispatch_combine_tokens_per_s", "value": value,
        "unit": "tokens/s", "n_gpus": R, "steps": iters, "warmup": warm,
        "ms_per_step": sec * 1e3, "us_per_layer": sec * 1e6, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3+bf16" if w["fp8"] else "bf16",
        "data": "synthetic",
        "config": {"workload": f"{w['name']}: {w['desc']}", "tokens_per_rank": w["T"],
                   "hidden": w["H"], "experts": w["E"], "topk": w["K"], "ranks": R},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"{iters} full dispatch+combine layers of all {R} ranks' work "
                                   f"in one process (torch CPU ops, {cores} threads)"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)
    return 0


# ----------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------
class _Solo:
    def rank(self):
        return 0

    def size(self):
        return 1


def run_ours(args):
    import torch
    import torch.distributed as dist
    from mooncake_b200 import Buffer, ep

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world == 1:
        # not under a launcher: start one process per GPU on this node
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1",
               "--master-port", str(29500 + os.getpid() % 1000), os.path.abspath(__file__)] + sys.argv[1:]
        return subprocess.call(cmd)
    R = world
    assert R == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if R > 1:
        # a short collective timeout: a rendezvous mismatch must fail in a minute, not in ten
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))
        group = dist.group.WORLD
    else:
        group = _Solo()

    w = workload(args)
    T, H, E, K = w["T"], w["H"], w["E"], w["K"]
    assert E % R == 0
    L, M = E // R, T
    inactive = args.inactive_rank
    i_am_out = (rank == inactive)

    x_h, idx_h, w_h = make_inputs(w, rank)
    x_h, idx_h, w_h = x_h.pin_memory(), idx_h.pin_memory(), w_h.pin_memory()
    x, idx, wts = x_h.to(dev), idx_h.to(dev), w_h.to(dev)
    active = torch.ones(R, dtype=torch.int32, device=dev)
    if inactive >= 0:
        active[inactive] = 0
    timeout_us = 2_000_000

    nbytes = Buffer.get_ep_buffer_size_hint(M, H, R, E)
    buf = Buffer(group, nbytes)
    if args.force_staged:
        buf.runtime.set_option("force_staged", 1)
    flush = torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.int32, device=dev)
    sync_word = torch.zeros(1, device=dev)
    y = torch.empty((L, R * M, H), dtype=torch.bfloat16, device=dev)
    out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    out_h = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
    cnt_h = torch.empty((L,), dtype=torch.int32).pin_memory()
    S = H // 128

    def expert(recv):
        """Mock expert, outside every timed region: dequantise, scale by (1 + e/16)."""
        e = (rank * L + torch.arange(L, device=dev, dtype=torch.float32)).view(L, 1, 1)
        f = (1.0 + e / 16.0).to(torch.bfloat16)
        if w["fp8"]:
            q, sc = recv
            v = q.view(L, R * M, S, 128).to(torch.bfloat16) * sc.unsqueeze(-1).to(torch.bfloat16)
            torch.mul(v.view(L, R * M, H), f, out=y)
        else:
            torch.mul(recv, f, out=y)
        return y

    def align_ranks():
        if R > 1:
            dist.all_reduce(sync_word)  # device-side rendezvous, keeps the ranks' steps aligned

    def step(ev=None):
        if i_am_out:
            # inactive for the EP exchange only: it still takes part in the
            # group's rendezvous collectives, or the others would wait for it
            align_ranks()
            align_ranks()
            return None
        if not args.no_flush:
            flush.zero_()
        align_ranks()
        if ev:
            ev[0].record()
        recv, cnt, handle, _, _ = buf.dispatch(x, idx, active, M, E, timeout_us, use_fp8=w["fp8"])
        if ev:
            ev[1].record()
        yy = expert(recv)
        if not args.no_flush:
            flush.zero_()
        align_ranks()
        if ev:
            ev[2].record()
        buf.combine(yy, idx, wts, active, timeout_us, handle, out=out)
        if ev:
            ev[3].record()
        return cnt

    def barrier():
        if R > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    barrier()

    # correctness inside the bench: expert = x * (1 + e/16) => closed form for the result
    if not i_am_out:
        f = 1.0 + idx.clamp_min(0).float() / 16.0
        keep = (idx >= 0)
        if inactive >= 0:
            keep &= (idx // L) != inactive
        ref = x.float() * (wts * f * keep).sum(dim=1, keepdim=True)
        err = float((out.float() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
        tol = 0.1 if w["fp8"] else 2e-2  # FP8 quantisation error dominates in the first case
        assert err < tol, f"bench self-check failed: rel err {err}"
        assert buf.runtime.status() == 0

    # ---- timed region: exactly K steps -------------------------------------------------
    K_steps = args.steps
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(K_steps)]
    sampler = ClockSampler(local_rank) if rank == 0 else None
    barrier()
    launches0 = ep.kernel_launch_count()
    if sampler:
        sampler.start()
    t_wall0 = time.perf_counter()
    for i in range(K_steps):
        step(evs[i])
    barrier()
    t_wall = time.perf_counter() - t_wall0
    launches = ep.kernel_launch_count() - launches0
    if i_am_out:
        td = torch.zeros(K_steps, device=dev)
        tc = torch.zeros(K_steps, device=dev)
    else:
        td = torch.tensor([e[0].elapsed_time(e[1]) for e in evs], device=dev)  # ms
        tc = torch.tensor([e[2].elapsed_time(e[3]) for e in evs], device=dev)
    if R > 1:
        dist.all_reduce(td, op=dist.ReduceOp.MAX)  # critical path: slowest rank per step
        dist.all_reduce(tc, op=dist.ReduceOp.MAX)
    layer_ms = (td + tc)
    ms_per_step = float(layer_ms.mean())
    p50 = float(layer_ms.median())

    # ---- per-kernel device times (events around every launch, kernels serialised) --------
    ep.set_kernel_timing(True)
    n_k = min(K_steps, 30)
    for _ in range(n_k):
        step()
    barrier()
    ktimes = ep.drain_kernel_times()
    ep.set_kernel_timing(False)
    # the sampler covers the timed region and the per-kernel pass that follows it
    # (same steps, same load); the timed region alone is too short for more than a
    # couple of nvidia-smi samples
    clocks = sampler.stop() if sampler else None

    # ---- end to end: host buffers in, host buffers out ------------------------------------
    e2e_times = []
    h2d = x_h.numel() * 2 + idx_h.numel() * 8 + w_h.numel() * 4
    d2h = out_h.numel() * 2 + cnt_h.numel() * 4
    for i in range(args.e2e_steps + 3):
        if i_am_out:
            align_ranks()
            align_ranks()
            continue
        align_ranks()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        x.copy_(x_h, non_blocking=True)
        idx.copy_(idx_h, non_blocking=True)
        recv, cnt, handle, _, _ = buf.dispatch(x, idx, active, M, E, timeout_us, use_fp8=w["fp8"])
        cnt_h.copy_(cnt, non_blocking=True)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        yy = expert(recv)
        align_ranks()
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        wts.copy_(w_h, non_blocking=True)
        buf.combine(yy, idx, wts, active, timeout_us, handle, out=out)
        out_h.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
        t3 = time.perf_counter()
        if i >= 3:
            e2e_times.append((t1 - t0) + (t3 - t2))
    e2e_t = torch.tensor(e2e_times if e2e_times else [0.0] * args.e2e_steps, device=dev)
    if R > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_sec = float(e2e_t.mean())

    # ---- roofline ----------------------------------------------------------------------------
    sel = int((idx >= 0).sum())
    n_active = R - (1 if inactive >= 0 else 0)
    tokens_total = T * n_active
    alg = algorithmic_bytes(w, R, sel)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_note = "of measured" if "hbm_gbs" in peaks else "of fallback"
    kern = {}
    for name, (n, ms) in ktimes.items():
        us = ms * 1e3 / max(n, 1)
        kern[name] = {"launches_per_step": n / max(n_k, 1), "avg_us": us,
                      "alg_bytes": alg.get(name), "share": None}
    tot = sum(v["avg_us"] * v["launches_per_step"] for v in kern.values()) or 1.0
    for v in kern.values():
        v["share"] = v["avg_us"] * v["launches_per_step"] / tot
    dom = max(kern, key=lambda k: kern[k]["share"]) if kern else None
    traffic = None
    try:
        tr = json.load(open(os.path.join(ROOT, "profiles", "ncu_traffic.json")))
        ent = tr.get(f"{w['name']}:{R}:{dom}")
        if ent:
            traffic = ent["dram_bytes_per_launch"]
    except Exception:
        pass
    roofline = None
    if dom and kern[dom]["alg_bytes"]:
        ach = kern[dom]["alg_bytes"] / (kern[dom]["avg_us"] * 1e-6) / 1e9
        roofline = {"bound": "hbm", "kernel": dom, "achieved": ach, "peak": hbm_peak,
                    "unit": "GB/s", "frac": ach / hbm_peak, "traffic": traffic,
                    "peak_source": peak_note, "alg_bytes_per_launch": kern[dom]["alg_bytes"],
                    "avg_us": kern[dom]["avg_us"]}
    nvlink = None
    if R > 1:
        payload_d = ((H + 4 * S) if w["fp8"] else 2 * H) + 16
        remote = sel * (R - 1) / R  # uniform-routing expectation; egress == ingress
        nv_bytes = remote * payload_d + remote * 2 * H
        t_roof_us = nv_bytes / 900e9 * 1e6
        nvlink = {"bytes_per_gpu_per_layer": nv_bytes, "gbs_per_gpu": nv_bytes / (ms_per_step * 1e-3) / 1e9,
                  "peak_gbs_per_direction": 900.0, "frac_of_peak": t_roof_us / (ms_per_step * 1e3),
                  "roofline_us": t_roof_us}
        if roofline is not None:
            roofline["note"] = "per-kernel figure against HBM; the layer-level NVLink figure is in `nvlink`"

    if rank != 0:
        if R > 1:
            dist.destroy_process_group()
        return 0

    cpu_baseline = None
    if R == 1 and not args.no_cpu_baseline:
        torch.set_num_threads(max(1, (os.cpu_count() or 1)))
        sec, iters, _ = cpu_layer_seconds(w, 1, budget_s=12.0)
        cpu_baseline = {"value": T / sec, "unit": "tokens/s", "cores": torch.get_num_threads(),
                        "kind": "port",
                        "sample": f"{iters} dispatch+combine layers of this workload at 1 rank "
                                  f"({sec * 1e3:.1f} ms each), CPU restatement of the reference's "
                                  "torch path"}

    value = tokens_total / (ms_per_step * 1e-3)
    line = {
        "metric": "ep_dispatch_combine_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": R, "steps": K_steps, "warmup": warm, "ms_per_step": ms_per_step,
        "us_per_layer": ms_per_step * 1e3, "us_per_layer_p50": p50 * 1e3,
        "dispatch_us": float(td.mean()) * 1e3, "combine_us": float(tc.mean()) * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3+bf16" if w["fp8"] else "bf16", "data": "synthetic",
        "config": {"workload": f"{w['name']}: {w['desc']}", "tokens_per_rank": T, "hidden": H,
                   "experts": E, "experts_per_rank": L, "topk": K, "ranks": R,
                   "l2": ("NOT FLUSHED (diagnosis run)" if args.no_flush else
                          f"flushed before every dispatch and every combine ({L2_FLUSH_BYTES >> 20} MiB write)"),
                   "timing": "CUDA events around dispatch and around combine, max over ranks per step, mean over steps",
                   "inactive_rank": inactive},
        "clocks": clocks, "gpu_launches": int(launches),
        "launches_per_step": launches / max(K_steps, 1),
        "wall_s_timed_region": t_wall,
        "e2e": {"value": tokens_total / e2e_sec if e2e_sec > 0 else None, "unit": "tokens/s",
                "us_per_layer": e2e_sec * 1e6, "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h),
                "how": "host wall clock around [H2D x, idx -> dispatch -> D2H recv_count] + "
                       "[H2D weights -> combine -> D2H combined_x], pinned host memory"},
        "roofline": roofline, "nvlink": nvlink, "kernels": kern, "cpu_baseline": cpu_baseline,
    }
    print(json.dumps(line), flush=True)
    if R > 1:
        dist.destroy_process_group()
    return 0


def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
