#!/usr/bin/env python
"""EP dispatch + combine benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4|c5]
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
    "c1": dict(T=128, H=2048, E=16, K=4, fp8=False, routing="softmax",
               desc="the CPU-runnable case: 128 tok/rank, hidden 2048, 16 experts, top-4 of softmax "
                    "gate logits, bf16 dispatch, bf16 combine"),
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
    ap.add_argument("--zero-copy", action="store_true",
                    help="headline run with zero-copy combine: the mock expert writes into the "
                         "buffer get_next_combine_buffer returns (default: reported beside the "
                         "headline in `zero_copy_combine`)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the secondary measurements (zero-copy figure, prefill block at N=1)")
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
    elif w["routing"] == "softmax":
        scores = torch.softmax(torch.randn((T, E), generator=g), dim=-1)
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
    """Bytes one rank must move per launch of each kernel, from the workload alone
    (sel = valid (token, expert) selections of the rank; a rank receives about
    what it sends)."""
    T, H, K = w["T"], w["H"], w["K"]
    S = H // 128
    payload = (H + 4 * S) if w["fp8"] else 2 * H   # per (token, selected expert)
    b = {}
    # single rank: x read once, packed outputs written once; combine gathers and writes once
    b["ep_dispatch_send_direct"] = T * 2 * H + sel * payload + 8 * T * K + 4 * sel
    b["ep_combine_reduce_direct"] = sel * 2 * H + T * 2 * H + 12 * T * K
    # group: rows go straight to their final place (one write per selection, local
    # or over NVLink); the receive duty only moves the small side messages
    remote = sel * (R - 1) / max(R, 1)
    b["ep_dispatch_send"] = T * 2 * H + sel * (payload + 16)
    b["ep_dispatch_recv"] = 2 * remote * (4 * S + 16 if w["fp8"] else 16)
    b["ep_dispatch"] = b["ep_dispatch_send"] + b["ep_dispatch_recv"]
    # combine: rows peers will ask for are copied into symmetric memory (read +
    # write), every token's K rows are read once and one row is written
    b["ep_combine_publish"] = 2 * remote * 2 * H
    b["ep_combine_reduce"] = sel * 2 * H + T * 2 * H + 12 * T * K
    b["ep_combine"] = b["ep_combine_publish"] + b["ep_combine_reduce"]
    return b


def nvlink_bytes(w, R, inactive=-1, idx_all=None):
    """Bytes that must cross NVLink per layer, from the actual routing of all ranks
    (`idx_all[r]` = rank r's top-k indices; regenerated from the seeds when not
    given): per GPU, egress and ingress of dispatch (payload of the
    reference's accounting: fp8 H + 4*H/128 + 16, bf16 2H per selection,
    mooncake-wheel/tests/test_mooncake_ep.py:117-122) and of combine (2H per
    selection). The roofline time is the largest of the four per phase, summed."""
    T, H, E, K = w["T"], w["H"], w["E"], w["K"]
    L = E // R
    pd = (H + 4 * (H // 128) + 16) if w["fp8"] else 2 * H
    pc = 2 * H
    d_out, d_in = [0] * R, [0] * R
    for r in range(R):
        if r == inactive:
            continue
        idx = idx_all[r] if idx_all is not None else make_inputs(w, r)[1]
        owner = (idx.clamp_min(0) // L)
        valid = idx >= 0
        for o in range(R):
            if o == r or o == inactive:
                continue
            n = int((valid & (owner == o)).sum())
            d_out[r] += n
            d_in[o] += n
    # combine mirrors dispatch: what a rank received it serves back, what it sent it fetches
    disp = max(max(d_out), max(d_in)) * pd
    comb = max(max(d_out), max(d_in)) * pc
    mean = sum(d_out) / max(1, R - (1 if inactive >= 0 else 0))
    return {"dispatch_bytes_max_gpu": disp, "combine_bytes_max_gpu": comb,
            "selections_remote_max_gpu": max(max(d_out), max(d_in)),
            "selections_remote_mean_gpu": mean,
            "roofline_us": (disp + comb) / 900e9 * 1e6}


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


def config_of(w, R, args):
    """The workload, spelled the same way by both arms."""
    return {"workload": f"{w['name']}: {w['desc']}", "tokens_per_rank": w["T"], "hidden": w["H"],
            "experts": w["E"], "experts_per_rank": w["E"] // R, "topk": w["K"], "ranks": R,
            "routing": w["routing"], "dispatch_payload": "fp8_e4m3" if w["fp8"] else "bf16",
            "inactive_rank": args.inactive_rank}


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
        "data": "synthetic", "config": config_of(w, R, args),
        "method": {"l2": "not applicable (host memory)",
                   "timing": "time.perf_counter around dispatch and around combine of all ranks"},
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


HOST_HIDE_CYCLES = 400_000  # ~200 us of device idle time at 1.9 GHz, queued ahead of each timed call


class Layer:
    """One rank's dispatch + combine on fixed synthetic inputs, with everything
    the timed loop needs allocated up front."""

    def __init__(self, args, w, group, rank, R, dev, zero_copy):
        import torch
        from mooncake_b200 import Buffer
        self.torch = torch
        self.args, self.w, self.rank, self.R, self.dev = args, w, rank, R, dev
        self.zero_copy = zero_copy
        T, H, E, K = w["T"], w["H"], w["E"], w["K"]
        self.L, self.M, self.S = E // R, T, H // 128
        self.x_h, self.idx_h, self.w_h = [t.pin_memory() for t in make_inputs(w, rank)]
        self.x, self.idx, self.wts = self.x_h.to(dev), self.idx_h.to(dev), self.w_h.to(dev)
        self.active = torch.ones(R, dtype=torch.int32, device=dev)
        self.inactive = args.inactive_rank
        if self.inactive >= 0:
            self.active[self.inactive] = 0
        self.i_am_out = rank == self.inactive
        self.rendezvous_launches = 0
        self.timeout_us = 2_000_000
        nbytes = Buffer.get_ep_buffer_size_hint(self.M, H, R, E) if (R > 1 or args.force_staged) else 0
        self.buf = Buffer(group, nbytes)
        if args.force_staged:
            self.buf.runtime.set_option("force_staged", 1)
        self.y = None if zero_copy else torch.empty((self.L, R * self.M, H), dtype=torch.bfloat16,
                                                    device=dev)
        self.out = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
        e = (rank * self.L + torch.arange(self.L, device=dev, dtype=torch.float32)).view(self.L, 1, 1)
        self.factor = (1.0 + e / 16.0).to(torch.bfloat16)

    def expert(self, recv, handle):
        """Mock expert, outside every timed region: dequantise, scale by (1 + e/16).
        With zero copy it writes into the buffer the next combine call reads."""
        torch, w = self.torch, self.w
        H = w["H"]
        y = self.buf.get_next_combine_buffer(handle) if self.zero_copy else self.y
        if w["fp8"]:
            q, sc = recv
            v = q.view(self.L, -1, self.S, 128).to(torch.bfloat16) * sc.unsqueeze(-1).to(torch.bfloat16)
            torch.mul(v.view(self.L, -1, H), self.factor, out=y)
        else:
            torch.mul(recv, self.factor, out=y)
        return y

    def dispatch(self):
        return self.buf.dispatch(self.x, self.idx, self.active, self.M, self.w["E"], self.timeout_us,
                                 use_fp8=self.w["fp8"])

    def combine(self, y, handle):
        return self.buf.combine(y, self.idx, self.wts, self.active, self.timeout_us, handle,
                                zero_copy=self.zero_copy, out=self.out)

    def check(self):
        """Closed form: expert e multiplies by (1 + e/16)."""
        if self.i_am_out:
            return
        torch, w = self.torch, self.w
        f = 1.0 + self.idx.clamp_min(0).float() / 16.0
        keep = (self.idx >= 0)
        if self.inactive >= 0:
            keep &= (self.idx // self.L) != self.inactive
        ref = self.x.float() * (self.wts * f * keep).sum(dim=1, keepdim=True)
        if ref.numel() == 0:
            return
        err = float((self.out.float() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
        tol = 0.1 if w["fp8"] else 2e-2  # FP8 quantisation error dominates in the first case
        assert err < tol, f"bench self-check failed: rel err {err}"
        assert self.buf.runtime.status() == 0


def timed_steps(layer, n_steps, n_warm, flush, sync, hide_host):
    """n_warm untimed and n_steps timed layers. Returns per-step (dispatch ms,
    combine ms) lists of this rank (zeros for a rank that sits out)."""
    import torch
    import torch.distributed as dist
    R = layer.R

    def align():
        if R > 1:
            # rendezvous of the ranks' streams: a collective keeps the hosts in step but
            # completes a few microseconds apart on different ranks, so the library's own
            # device-side barrier (every rank leaves within about one NVLink latency of the
            # others) follows it for the ranks that take part in the exchange
            dist.all_reduce(sync)
            if not layer.i_am_out:
                layer.buf.runtime.barrier(torch.cuda.current_stream().cuda_stream,
                                          layer.active.data_ptr())
                layer.rendezvous_launches += 1

    def step(ev):
        if layer.i_am_out:
            # inactive for the EP exchange only: it still takes part in the
            # group's rendezvous collectives, or the others would wait for it
            align()
            align()
            return
        if flush is not None:
            flush.zero_()
        align()
        if hide_host:
            # idle time on the device while the host runs ahead: the Python and the
            # launch of the timed call are queued before the GPU reaches its events
            torch.cuda._sleep(HOST_HIDE_CYCLES)
        if ev:
            ev[0].record()
        recv, cnt, handle, _, _ = layer.dispatch()
        if ev:
            ev[1].record()
        y = layer.expert(recv, handle)
        if flush is not None:
            flush.zero_()
        align()
        if hide_host:
            torch.cuda._sleep(HOST_HIDE_CYCLES)
        if ev:
            ev[2].record()
        layer.combine(y, handle)
        if ev:
            ev[3].record()

    for _ in range(n_warm):
        step(None)
    if R > 1:
        dist.barrier()
    torch.cuda.synchronize()
    layer.check()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(n_steps)]
    if R > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(n_steps):
        step(evs[i])
    if R > 1:
        dist.barrier()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    if layer.i_am_out:
        return [0.0] * n_steps, [0.0] * n_steps, wall, step
    return ([e[0].elapsed_time(e[1]) for e in evs], [e[2].elapsed_time(e[3]) for e in evs], wall,
            step)


def elastic_block(w, layer, group, rank, R, dev, flush, sync, n_steps):
    """The same inputs through the elastic-style interface (`ElasticBuffer`: a token
    travels once per destination rank, flat receive rows, unweighted combine), bf16
    payloads, timed like the headline. Returns this rank's per-step times."""
    import torch
    import torch.distributed as dist
    from mooncake_b200.mooncake_elastic_buffer import ElasticBuffer
    T, H, E, K = w["T"], w["H"], w["E"], w["K"]
    buf = ElasticBuffer(group, num_max_tokens_per_rank=T, hidden=H, num_topk=K, num_gpu_timeout_secs=2)
    stream = torch.cuda.current_stream().cuda_stream

    def align():
        if R > 1:
            dist.all_reduce(sync)
            buf.runtime.barrier(stream, 0)
        # the wrapper allocates its outputs inside the call: a longer idle period hides that too
        torch.cuda._sleep(3 * HOST_HIDE_CYCLES)

    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(n_steps)]
    rows = 0
    for i in range(-3, n_steps):
        ev = evs[i] if i >= 0 else None
        if flush is not None:
            flush.zero_()
        align()
        if ev:
            ev[0].record()
        recv, _, _, handle, _ = buf.dispatch(layer.x, topk_idx=layer.idx, topk_weights=layer.wts,
                                             num_experts=E, num_max_tokens_per_rank=T, do_cpu_sync=False)
        if ev:
            ev[1].record()
        if flush is not None:
            flush.zero_()
        align()
        if ev:
            ev[2].record()
        out, _, _ = buf.combine(recv, handle)  # identity expert
        if ev:
            ev[3].record()
        if i == -1:
            torch.cuda.synchronize()
            rows = int(handle.psum_num_recv_tokens_per_scaleup_rank[-1])
            assert buf.runtime.status() == 0, "device-side anomaly in the elastic calls"
    torch.cuda.synchronize()
    td = [e[0].elapsed_time(e[1]) for e in evs]
    tc = [e[2].elapsed_time(e[3]) for e in evs]
    # per-kernel device times of the same calls (events around every launch)
    from mooncake_b200 import ep
    ep.set_kernel_timing(True)
    n_k = 10
    for _ in range(n_k):
        align()
        recv, _, _, handle, _ = buf.dispatch(layer.x, topk_idx=layer.idx, topk_weights=layer.wts,
                                             num_experts=E, num_max_tokens_per_rank=T, do_cpu_sync=False)
        align()
        buf.combine(recv, handle)
    if R > 1:
        dist.barrier()
    torch.cuda.synchronize()
    kt = {k: round(ms * 1e3 / max(n, 1), 2) for k, (n, ms) in ep.drain_kernel_times().items()
          if k != "ep_barrier"}
    ep.set_kernel_timing(False)
    buf.destroy()
    return td, tc, rows, kt


def elastic_nvlink_us(w, R, idx_all):
    """Link time of the elastic exchange on the busiest GPU: one bf16 row per (token,
    remote destination rank) each way, over 900 GB/s per direction."""
    L = w["E"] // R
    eg, ing = [0] * R, [0] * R
    for s, idx in enumerate(idx_all):
        ranks = torch_unique_ranks(idx, L, R)
        for d in range(R):
            if d != s:
                n = int(ranks[:, d].sum())
                eg[s] += n
                ing[d] += n
    rows = max(max(eg), max(ing))
    return 2 * rows * 2 * w["H"] / 900e9 * 1e6, rows


def torch_unique_ranks(idx, L, R):
    """[T, R] bool: does token t name an expert of rank r."""
    import torch
    out = torch.zeros((idx.shape[0], R), dtype=torch.bool)
    for k in range(idx.shape[1]):
        col = idx[:, k]
        ok = col >= 0
        out[torch.nonzero(ok).squeeze(1), (col[ok] // L)] = True
    return out


def summarise(td, tc, dev, R):
    """Per-step max over ranks (the critical path), then mean / p50 / p90 over steps."""
    import torch
    import torch.distributed as dist
    td = torch.tensor(td, device=dev)
    tc = torch.tensor(tc, device=dev)
    if R > 1:
        dist.all_reduce(td, op=dist.ReduceOp.MAX)
        dist.all_reduce(tc, op=dist.ReduceOp.MAX)
    layer_ms = td + tc
    q = lambda t, p: float(torch.quantile(t, p))  # noqa: E731
    return {"us_per_layer": float(layer_ms.mean()) * 1e3, "us_per_layer_p50": q(layer_ms, 0.5) * 1e3,
            "us_per_layer_p90": q(layer_ms, 0.9) * 1e3, "us_per_layer_max": float(layer_ms.max()) * 1e3,
            "dispatch_us": float(td.mean()) * 1e3,
            "dispatch_us_p50": q(td, 0.5) * 1e3, "combine_us": float(tc.mean()) * 1e3,
            "combine_us_p50": q(tc, 0.5) * 1e3}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from mooncake_b200 import ep

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
    inactive = args.inactive_rank
    flush = None if args.no_flush else torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.int32, device=dev)
    sync_word = torch.zeros(1, device=dev)

    layer = Layer(args, w, group, rank, R, dev, zero_copy=args.zero_copy)
    warm = max(args.warmup, 3)
    K_steps = args.steps

    # ---- timed region: exactly K steps -------------------------------------------------
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    launches0 = ep.kernel_launch_count()
    layer.rendezvous_launches = 0
    td, tc, t_wall, step = timed_steps(layer, K_steps, warm, flush, sync_word, hide_host=True)
    # launches of the timed steps alone (the warm-up steps launch the same kernels); the
    # rendezvous barrier between the event pairs is the bench's, not the hot path's
    launches = ((ep.kernel_launch_count() - launches0 - layer.rendezvous_launches)
                * K_steps // (K_steps + warm))
    main = summarise(td, tc, dev, R)
    ms_per_step = main["us_per_layer"] * 1e-3

    # ---- per-kernel device times (events around every launch, kernels serialised) --------
    ep.set_kernel_timing(True)
    n_k = min(K_steps, 30)
    for _ in range(n_k):
        step(None)
    if R > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ktimes = ep.drain_kernel_times()
    ep.set_kernel_timing(False)
    # the sampler covers the timed region and the per-kernel pass that follows it
    # (same steps, same load); the timed region alone is too short for more than a
    # couple of nvidia-smi samples
    clocks = sampler.stop() if sampler else None

    # ---- end to end: host buffers in, host buffers out ------------------------------------
    out_h = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
    cnt_h = torch.empty((layer.L,), dtype=torch.int32).pin_memory()
    e2e_times = []
    h2d = layer.x_h.numel() * 2 + layer.idx_h.numel() * 8 + layer.w_h.numel() * 4
    d2h = out_h.numel() * 2 + cnt_h.numel() * 4

    def align():
        if R > 1:
            dist.all_reduce(sync_word)

    for i in range(args.e2e_steps + 3):
        if layer.i_am_out:
            align()
            align()
            continue
        align()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        layer.x.copy_(layer.x_h, non_blocking=True)
        layer.idx.copy_(layer.idx_h, non_blocking=True)
        recv, cnt, handle, _, _ = layer.dispatch()
        cnt_h.copy_(cnt, non_blocking=True)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        yy = layer.expert(recv, handle)
        align()
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        layer.wts.copy_(layer.w_h, non_blocking=True)
        layer.combine(yy, handle)
        out_h.copy_(layer.out, non_blocking=True)
        torch.cuda.synchronize()
        t3 = time.perf_counter()
        if i >= 3:
            e2e_times.append((t1 - t0) + (t3 - t2))
    e2e_t = torch.tensor(e2e_times if e2e_times else [0.0] * args.e2e_steps, device=dev)
    if R > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_sec = float(e2e_t.mean())

    # ---- zero-copy combine beside the headline (same buffer, same inputs) ------------------
    zero_copy = None
    if R > 1 and not args.zero_copy and not args.no_extras:
        layer.zero_copy = True
        td2, tc2, _, _ = timed_steps(layer, max(10, K_steps // 2), 3, flush, sync_word, hide_host=True)
        layer.zero_copy = False
        z = summarise(td2, tc2, dev, R)
        zero_copy = {"us_per_layer": z["us_per_layer"], "us_per_layer_p50": z["us_per_layer_p50"],
                     "combine_us": z["combine_us"], "combine_us_p50": z["combine_us_p50"],
                     "how": "expert outputs written into get_next_combine_buffer, "
                            "combine(zero_copy=True)"}

    # ---- roofline ----------------------------------------------------------------------------
    sel = int((layer.idx >= 0).sum())
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

    def kernel_table(kt, n_steps, alg_bytes):
        kern = {}
        for name, (n, ms) in kt.items():
            us = ms * 1e3 / max(n, 1)
            ab = alg_bytes.get(name)
            kern[name] = {"launches_per_step": n / max(n_steps, 1), "avg_us": us, "alg_bytes": ab,
                          "hbm_frac": (ab / (us * 1e-6) / 1e9 / hbm_peak) if ab else None,
                          "share": None}
        tot = sum(v["avg_us"] * v["launches_per_step"] for v in kern.values()) or 1.0
        for v in kern.values():
            v["share"] = v["avg_us"] * v["launches_per_step"] / tot
        return kern

    ktimes.pop("ep_barrier", None)  # the rendezvous between the timed calls
    kern = kernel_table(ktimes, n_k, alg)
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
    idx_all = None
    if R > 1:
        gathered = [torch.empty_like(layer.idx) for _ in range(R)]
        dist.all_gather(gathered, layer.idx)
        idx_all = [g.cpu() for g in gathered]
    if R > 1 and rank == 0:
        nv = nvlink_bytes(w, R, inactive, idx_all)
        nv_bytes = nv["dispatch_bytes_max_gpu"] + nv["combine_bytes_max_gpu"]
        nvlink = dict(nv)
        nvlink.update({"bytes_max_gpu_per_layer": nv_bytes,
                       "gbs_max_gpu": nv_bytes / (ms_per_step * 1e-3) / 1e9,
                       "peak_gbs_per_direction": 900.0,
                       "frac_of_peak": nv["roofline_us"] / (ms_per_step * 1e3),
                       "frac_of_peak_p50": nv["roofline_us"] / main["us_per_layer_p50"],
                       "how": "bytes the busiest GPU must send or receive per phase (from all ranks' "
                              "routing) / 900 GB/s, over the measured layer time"})
        if zero_copy:
            zero_copy["nvlink_frac_of_peak"] = nv["roofline_us"] / zero_copy["us_per_layer"]
        if roofline is not None:
            roofline["note"] = "per-kernel figure against HBM; the layer-level NVLink figure is in `nvlink`"

    # ---- N = 1: the prefill shape beside the headline (the bandwidth-bound case) -----------
    prefill = None
    if R == 1 and w["name"] == "c2" and args.tokens is None and not args.no_extras \
            and not args.force_staged:
        del layer
        torch.cuda.empty_cache()
        w3 = dict(WORKLOADS["c3"])
        w3["name"] = "c3"
        l3 = Layer(args, w3, group, rank, R, dev, zero_copy=False)
        n3 = 20
        td3, tc3, _, step3 = timed_steps(l3, n3, 3, flush, sync_word, hide_host=True)
        p3 = summarise(td3, tc3, dev, R)
        ep.set_kernel_timing(True)
        for _ in range(10):
            step3(None)
        torch.cuda.synchronize()
        k3 = kernel_table(ep.drain_kernel_times(), 10,
                          algorithmic_bytes(w3, 1, int((l3.idx >= 0).sum())))
        ep.set_kernel_timing(False)
        sel3 = int((l3.idx >= 0).sum())
        layer_bytes = (w3["T"] * 2 * w3["H"] + sel3 * 2 * w3["H"] + 8 * w3["T"] * w3["K"] + 4 * sel3
                       + sel3 * 2 * w3["H"] + w3["T"] * 2 * w3["H"] + 12 * w3["T"] * w3["K"])
        prefill = {"workload": f"c3: {w3['desc']}", "steps": n3, **p3,
                   "tokens_per_s": w3["T"] / (p3["us_per_layer"] * 1e-6),
                   "alg_bytes_per_layer": layer_bytes,
                   "hbm_frac_layer": layer_bytes / (p3["us_per_layer"] * 1e-6) / 1e9 / hbm_peak,
                   "hbm_frac_layer_p50": layer_bytes / (p3["us_per_layer_p50"] * 1e-6) / 1e9 / hbm_peak,
                   "kernels": k3}
        del l3

    # ---- the elastic-style interface on the same inputs ------------------------------------
    elastic = None
    if not args.no_extras and inactive < 0 and not args.force_staged and w["T"] <= 1024:
        # an extra beside the headline: an argument or state error here (raised alike on every
        # rank, before anything is launched) must not cost the line its headline
        try:
            elayer = Layer(args, w, group, rank, R, dev, zero_copy=False) if prefill is not None else layer
            tde, tce, rows, ekt = elastic_block(w, elayer, group, rank, R, dev, flush, sync_word,
                                                max(10, K_steps // 2))
            ze = summarise(tde, tce, dev, R)
            elastic = {"us_per_layer": ze["us_per_layer"], "us_per_layer_p50": ze["us_per_layer_p50"],
                       "dispatch_us": ze["dispatch_us"], "combine_us": ze["combine_us"],
                       "rows_received_rank0": rows, "payload": "bf16", "kernel_us": ekt,
                       "how": "ElasticBuffer.dispatch(do_cpu_sync=False) + ElasticBuffer.combine on the "
                              "headline's inputs, identity expert, timed like the headline"}
            if R > 1 and rank == 0:
                us, nrows = elastic_nvlink_us(w, R, idx_all)
                elastic.update({"nvlink_roofline_us": us, "rows_busiest_gpu": nrows,
                                "nvlink_frac_of_peak": us / ze["us_per_layer"]})
        except (RuntimeError, AssertionError) as exc:
            elastic = {"error": str(exc)[:300]}

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
        "n_gpus": R, "steps": K_steps, "warmup": warm, "ms_per_step": ms_per_step, **main,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3+bf16" if w["fp8"] else "bf16", "data": "synthetic",
        "config": config_of(w, R, args),
        "method": {"l2": ("NOT FLUSHED (diagnosis run)" if args.no_flush else
                          f"flushed before every dispatch and every combine ({L2_FLUSH_BYTES >> 20} MiB write)"),
                   "timing": "CUDA events around Buffer.dispatch and around Buffer.combine on the calling "
                             "stream; before each timed call the ranks are released together by a "
                             "device-side barrier over NVLink and a fixed device-side idle period is "
                             "queued so the host's share of the call is not on the device's clock; max "
                             "over ranks per step; mean, p50 and p90 over steps",
                   "combine": "zero_copy=True" if args.zero_copy else "zero_copy=False",
                   "recv_x": "in place (symmetric memory)" if (R > 1 or args.force_staged) else
                             "caller's tensor (single rank)"},
        "clocks": clocks, "gpu_launches": int(launches),
        "launches_per_step": launches / max(K_steps, 1),
        "wall_s_timed_region": t_wall,
        "e2e": {"value": tokens_total / e2e_sec if e2e_sec > 0 else None, "unit": "tokens/s",
                "us_per_layer": e2e_sec * 1e6, "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h),
                "how": "host wall clock around [H2D x, idx -> dispatch -> D2H recv_count] + "
                       "[H2D weights -> combine -> D2H combined_x], pinned host memory"},
        "roofline": roofline, "nvlink": nvlink, "zero_copy_combine": zero_copy,
        "prefill_1gpu": prefill, "elastic": elastic, "kernels": kern, "cpu_baseline": cpu_baseline,
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
