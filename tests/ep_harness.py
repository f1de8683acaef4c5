"""Shared helpers of the GPU tests: seeded inputs for the benchmark shapes and
an in-process group that runs several logical ranks one after the other on one
GPU (all sends first, then all receives, so no kernel ever waits for a later
launch)."""
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
                hard_timeout_ms: int = 2000) -> List[Buffer]:
    """R logical ranks on the current device, mapped to each other directly."""
    bufs = []
    for r in range(R):
        b = Buffer.__new__(Buffer)
        b.rank, b.group_size, b.group, b.backend = r, R, None, None
        b.num_ep_buffer_bytes = num_bytes
        b.runtime = ep.Buffer(r, R, num_bytes, False)
        b._use_fallback = False
        b._warned_active_ranks = True
        b.runtime.set_option("hard_timeout_ms", hard_timeout_ms)
        if force_staged:
            b.runtime.set_option("force_staged", 1)
        bufs.append(b)
    bases = [b.runtime.local_base() for b in bufs]
    for b in bufs:
        b.runtime.set_peer_bases(bases)
    return bufs


def run_dispatch(bufs, xs, idxs, M, E, use_fp8, active=None, timeout_us=200_000):
    """SEND on every participating rank, then RECV on every one. Returns per rank
    (recv_x, scales, recv_count, handle, active_ranks_tensor) or None."""
    R = len(bufs)
    act = [1] * R if active is None else list(active)
    pend = [None] * R
    for r in range(R):
        if not act[r]:
            continue
        ar = torch.tensor(act, dtype=torch.int32, device="cuda")
        rx, cnt, handle, _, hook = bufs[r].dispatch(xs[r].cuda(), idxs[r].cuda(), ar, M, E,
                                                     timeout_us, use_fp8=use_fp8,
                                                     return_recv_hook=True)
        pend[r] = (rx, cnt, handle, hook, ar)
    out = [None] * R
    for r in range(R):
        if pend[r] is None:
            continue
        rx, cnt, handle, hook, ar = pend[r]
        hook()
        out[r] = dict(recv_x=rx[0] if use_fp8 else rx, scales=rx[1] if use_fp8 else None,
                      recv_count=cnt, handle=handle, active=ar)
    torch.cuda.synchronize()
    return out


def run_combine(bufs, ys, idxs, ws, handles, active=None, timeout_us=200_000):
    R = len(bufs)
    act = [1] * R if active is None else list(active)
    pend = [None] * R
    for r in range(R):
        if not act[r]:
            continue
        ar = torch.tensor(act, dtype=torch.int32, device="cuda")
        di, dw = idxs[r].cuda(), ws[r].cuda()  # read again by the receive phase: keep alive
        out, _, hook = bufs[r].combine(ys[r], di, dw, ar, timeout_us, handles[r],
                                       return_recv_hook=True)
        pend[r] = (out, hook, ar, di, dw)
    res = [None] * R
    for r in range(R):
        if pend[r] is None:
            continue
        out, hook, ar = pend[r][:3]
        hook()
        res[r] = (out, ar)
    torch.cuda.synchronize()
    return res


def mock_expert(recv_bf16: torch.Tensor, rank: int, L: int) -> torch.Tensor:
    """y = x * (1 + e/16) in fp32, rounded to bf16 (the mock expert of the CPU-runnable case)."""
    e = (rank * L + torch.arange(L, device=recv_bf16.device)).float().view(L, 1, 1)
    return (recv_bf16.float() * (1.0 + e / 16.0)).to(torch.bfloat16)
