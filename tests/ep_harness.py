"""Shared helpers of the GPU tests: seeded inputs for the benchmark shapes and
an in-process group of several logical ranks on one GPU. In a group the ranks'
kernels wait for one another (an expert's owner answers every source), so the
logical ranks never run as separate launches: each prepares its call
("defer_launch") and `ep.launch_deferred` starts all of them as ONE cooperative
launch. Phases that wait for nothing launched later (a receive phase after
every send phase has completed) run rank by rank."""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from mooncake_b200 import ep
from mooncake_b200.mooncake_ep_buffer import Buffer


def routing(kind: str, T: int, E: int, K: int, g: torch.Generator) -> torch.Tensor:
    """Routing generators with the distributions of the reference's benchmark
    (mooncake-ep/benchmarks/ep_benchmark/routing.py:19-43 uniform, :104-146 zipf)."""
    if kind == "uniform":
        scores = torch.randn((T, E), generator=g)
    elif kind == "softmax":
        scores = torch.softmax(torch.randn((T, E), generator=g), dim=-1)
    elif kind.startswith("zipf"):
        alpha = float(kind[4:] or 1.2)
        logp = -alpha * torch.log(torch.arange(1, E + 1, dtype=torch.float32))
        logp = logp - torch.logsumexp(logp, dim=0)
        u = torch.rand((T, E), generator=g).clamp(min=1e-20)
        scores = logp.unsqueeze(0) - torch.log(-torch.log(u))
    else:
        raise ValueError(kind)
    return torch.topk(scores, K, dim=-1)[1].to(torch.int64).contiguous()


def make_rank_inputs(seed: int, rank: int, T: int, H: int, E: int, K: int, kind: str = "uniform",
                     n_mask: int = 0):
    g = torch.Generator().manual_seed(seed * 7919 + rank)
    x = torch.randn((T, H), generator=g).to(torch.bfloat16)
    idx = routing(kind, T, E, K, g)
    w = torch.softmax(torch.rand((T, K), generator=g), dim=-1).float().contiguous()
    for _ in range(n_mask if T else 0):
        idx[int(torch.randint(0, T, (1,), generator=g)), int(torch.randint(0, K, (1,), generator=g))] = -1
    return x, idx, w


class FakeGroup:
    """Stands in for a torch.distributed group where no collective is needed."""

    def __init__(self, rank: int, size: int):
        self._r, self._s = rank, size

    def rank(self):
        return self._r

    def size(self):
        return self._s


def local_group(R: int, num_bytes: int, force_staged: bool = True,
                hard_timeout_ms: int = 2000, recv_in_place: bool = True) -> List[Buffer]:
    """R logical ranks on the current device, mapped to each other directly."""
    bufs = []
    for r in range(R):
        b = Buffer.__new__(Buffer)
        b.rank, b.group_size, b.group, b.backend = r, R, None, None
        b.num_ep_buffer_bytes = num_bytes
        b.recv_in_place = recv_in_place
        b._views = {}
        b.runtime = ep.Buffer(r, R, num_bytes, False)
        b._use_fallback = False
        b._warned_active_ranks = True
        b.runtime.set_option("hard_timeout_ms", hard_timeout_ms)
        if force_staged:
            b.runtime.set_option("force_staged", 1)
        if R > 1 or force_staged:
            b.runtime.set_option("defer_launch", 1)
        bufs.append(b)
    connect_local_group(bufs)
    return bufs


def connect_local_group(bufs: List[Buffer], available: Optional[List[int]] = None) -> None:
    """(Re)connect an in-process group: what `Buffer.connect` does with memory
    handles and an all-gather, done with base pointers. Also brings the ranks'
    call counters back in step (membership refresh)."""
    bases = [b.runtime.local_base() for b in bufs]
    for b in bufs:
        b.runtime.set_peer_bases(bases, available)


def run_dispatch(bufs, xs, idxs, M, E, use_fp8, active=None, timeout_us=200_000, mode="hook"):
    """Dispatch on every participating rank. mode "hook": send phase of all ranks
    (one launch), then every rank's receive phase from its hook; mode "sync": no
    hook - small batches then run both phases in the one launch. Returns per rank
    a dict (recv_x, scales, recv_count, handle, active) or None."""
    R = len(bufs)
    act = [1] * R if active is None else list(active)
    pend = [None] * R
    for r in range(R):
        if not act[r]:
            continue
        ar = torch.tensor(act, dtype=torch.int32, device="cuda")
        dx, di = xs[r].cuda(), idxs[r].cuda()
        rx, cnt, handle, _, hook = bufs[r].dispatch(dx, di, ar, M, E, timeout_us, use_fp8=use_fp8,
                                                     return_recv_hook=(mode == "hook"))
        pend[r] = (rx, cnt, handle, hook, ar, dx, di)
    ep.launch_deferred([bufs[r].runtime for r in range(R) if pend[r] is not None])
    out = [None] * R
    for r in range(R):
        if pend[r] is None:
            continue
        rx, cnt, handle, hook, ar = pend[r][:5]
        if hook:
            hook()
        out[r] = dict(recv_x=rx[0] if use_fp8 else rx, scales=rx[1] if use_fp8 else None,
                      recv_count=cnt, handle=handle, active=ar)
    torch.cuda.synchronize()
    return out


def run_combine(bufs, ys, idxs, ws, handles, active=None, timeout_us=200_000, mode="hook",
                zero_copy=False):
    """Combine on every participating rank. mode "hook": every rank's first phase
    (it waits for nobody), then every rank's reduce from its hook; mode "sync":
    both phases of all ranks in one launch. With zero_copy the expert outputs are
    first written into `get_next_combine_buffer`."""
    R = len(bufs)
    act = [1] * R if active is None else list(active)
    pend = [None] * R
    for r in range(R):
        if not act[r]:
            continue
        ar = torch.tensor(act, dtype=torch.int32, device="cuda")
        di, dw = idxs[r].cuda(), ws[r].cuda()  # read again by the receive phase: keep alive
        y = ys[r]
        if zero_copy:
            bufs[r].get_next_combine_buffer(handles[r]).copy_(y)
            y = torch.empty_like(y)  # only its shape is looked at
        out, _, hook = bufs[r].combine(y, di, dw, ar, timeout_us, handles[r], zero_copy=zero_copy,
                                       return_recv_hook=(mode == "hook"))
        pend[r] = (out, hook, ar, di, dw, y)
    ep.launch_deferred([bufs[r].runtime for r in range(R) if pend[r] is not None])
    res = [None] * R
    for r in range(R):
        if pend[r] is None:
            continue
        out, hook, ar = pend[r][:3]
        if hook:
            hook()
        res[r] = (out, ar)
    torch.cuda.synchronize()
    return res


def mock_expert(recv_bf16: torch.Tensor, rank: int, L: int) -> torch.Tensor:
    """y = x * (1 + e/16) in fp32, rounded to bf16 (the mock expert of the CPU-runnable case)."""
    e = (rank * L + torch.arange(L, device=recv_bf16.device)).float().view(L, 1, 1)
    return (recv_bf16.float() * (1.0 + e / 16.0)).to(torch.bfloat16)
