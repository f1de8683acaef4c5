"""CPU oracle for Mooncake EP `Buffer.dispatch` / `Buffer.combine`.

TEST INFRASTRUCTURE ONLY: imported by `tests/`, by `__graft_entry__.smoke()`
and by the CPU-baseline legs of `bench.py`. The product package never imports
it and has no CPU fallback.

It restates, for all ranks of a group at once and in one process, what the
reference computes (paths relative to the Mooncake tree):

* canonical receive order: source rank ascending, token ascending - the order
  of the reference's torch path (mooncake-wheel/mooncake/mooncake_ep_buffer.py:
  787-818) and one of the orders its CUDA kernel may produce
  (mooncake-ep/src/mooncake_ep_kernel.cu:274,430);
* `layout_range = (begin << 32) | count` (mooncake_ep_kernel.cu:433; the
  torch path stores a literal 0 for empty sources, mooncake_ep_buffer.py:817);
* FP8 payload and scales with the kernel's formula (mooncake_ep_kernel.cu:
  184,239-264) or, with `arith="fallback"`, the torch path's
  (mooncake_ep_buffer.py:693-703) - they differ in the last bit of the scale;
* combine as fp32 FMA in top-k order with one bf16 rounding
  (mooncake_ep_kernel.cu:715-752) or, with `arith="fallback"`, the torch path's
  bf16 running sum (mooncake_ep_buffer.py:1012-1048).

Parity status: pinned against outputs of the reference's torch path generated
in a container that has the Mooncake sources (`tests/golden/`).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import build as _build

_LIB = None


def lib() -> ctypes.CDLL:
    """The C restatement (`ep_oracle.c`), compiled on first use."""
    global _LIB
    if _LIB is None:
        path = _build.build_oracle()
        L = ctypes.CDLL(path)
        L.ora_e4m3_from_f32.restype = ctypes.c_uint8
        L.ora_e4m3_from_f32.argtypes = [ctypes.c_float]
        L.ora_fp8_quant_rows.restype = None
        L.ora_fp8_quant_rows.argtypes = [ctypes.c_void_p, ctypes.c_int64,
                                         ctypes.c_int, ctypes.c_void_p,
                                         ctypes.c_void_p]
        for name, _ in (("ora_combine_reduce", 0), ("ora_combine_reduce_f32", 1)):
            fn = getattr(L, name)
            fn.restype = None
            fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                           ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                           ctypes.c_void_p]
        _LIB = L
    return _LIB


# --------------------------------------------------------------------------
# routing layout
# --------------------------------------------------------------------------
def routing_layout(topk_idx: torch.Tensor, num_experts: int,
                   num_ranks: int) -> Dict[str, torch.Tensor]:
    """Per-expert / per-rank counts, prefix offsets and per-entry slots.

    `slot[t, k]` is the number of tokens `t' < t` of this rank that select the
    same expert (each token counted once per expert), i.e. the position the
    (token, expert) message takes among this rank's messages for that expert
    in token-ascending order. Masked entries (`-1`,
    mooncake_ep_kernel.cu:273) and a repeated expert inside one token's list
    (counted once, as `.any(dim=1)` does in mooncake_ep_buffer.py:797-803) get
    slot -1.
    """
    T, K = topk_idx.shape
    E, R = num_experts, num_ranks
    L = E // R
    idx = topk_idx.to(torch.int64)
    sel = torch.zeros((T, E + 1), dtype=torch.int32)
    safe = torch.where(idx >= 0, idx, torch.full_like(idx, E))
    if T > 0:
        sel.scatter_(1, safe, 1)
    sel = sel[:, :E]
    excl = torch.cumsum(sel, dim=0, dtype=torch.int32) - sel  # exclusive, over tokens
    count = sel.sum(dim=0, dtype=torch.int32)
    slot = torch.full((T, K), -1, dtype=torch.int32)
    for k in range(K):
        e = idx[:, k]
        ok = e >= 0
        for kk in range(k):
            ok &= idx[:, kk] != e
        rows = torch.nonzero(ok).view(-1)
        slot[rows, k] = excl[rows, e[rows]]
    rank_count = count.view(R, L).sum(dim=1, dtype=torch.int32)
    per_rank = count.view(R, L)
    expert_prefix = (torch.cumsum(per_rank, dim=1, dtype=torch.int32) - per_rank).reshape(E)
    return dict(count=count, rank_count=rank_count, expert_prefix=expert_prefix,
                slot=slot)


# --------------------------------------------------------------------------
# FP8
# --------------------------------------------------------------------------
def fp8_quant(x: torch.Tensor, arith: str = "kernel"):
    """bf16 `[rows, H]` -> (e4m3 bytes as uint8 `[rows, H]`, fp32 scales `[rows, H/128]`)."""
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.size(1) % 128 == 0
    rows, H = x.shape
    x = x.contiguous()
    if arith == "fallback":
        # mooncake_ep_buffer.py:693-703, op for op
        xv = x.view(rows, -1, 128)
        amax = xv.abs().float().amax(dim=2).view(rows, -1).clamp(1e-4)
        q = (xv * (448.0 / amax.unsqueeze(2))).to(torch.float8_e4m3fn).view(rows, H)
        return q.view(torch.uint8), (amax / 448.0).view(rows, -1)
    q = torch.empty((rows, H), dtype=torch.uint8)
    s = torch.empty((rows, H // 128), dtype=torch.float32)
    if rows:
        lib().ora_fp8_quant_rows(x.data_ptr(), rows, H, q.data_ptr(), s.data_ptr())
    return q, s


def fp8_dequant(q_u8: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """e4m3 bytes + per-128 scales -> bf16, the way the reference's test helper
    casts back (mooncake-wheel/tests/ep_test_utils.py:50-53)."""
    rows, H = q_u8.shape
    f = q_u8.view(torch.float8_e4m3fn).to(torch.float32).view(rows, H // 128, 128)
    return (f * scales.view(rows, H // 128, 1)).view(rows, H).to(torch.bfloat16)


# --------------------------------------------------------------------------
# dispatch
# --------------------------------------------------------------------------
def dispatch(xs: Sequence[Optional[torch.Tensor]],
             topks: Sequence[Optional[torch.Tensor]],
             num_max_dispatch_tokens_per_rank: int, num_experts: int,
             use_fp8: bool, active: Optional[Sequence[int]] = None,
             arith: str = "kernel") -> List[Optional[dict]]:
    """All ranks' dispatch outputs.

    `xs[r]` is rank r's `[T_r, H]` bf16 input, `topks[r]` its `[T_r, K]` int64
    expert list. Ranks with `active[r] == 0` send nothing and receive nothing
    (their entry in the result is None): every receiver sees a count of 0 from
    them, as when the reference's wait loop leaves on the mask
    (mooncake_ep_kernel.cu:424-429).

    Per active rank the result holds `recv_x` `[L, R*M, H]` (uint8 e4m3 bytes
    or bf16), `scales` `[L, R*M, H/128]` fp32 (logical layout; fp8 only),
    `recv_count` `[L]` int32, `src_info` `[L, R*M]` int32, `layout_range`
    `[L, R]` int64. Rows at or beyond `recv_count` are zero / -1 here and
    unspecified in the product.
    """
    R = len(xs)
    M, E = num_max_dispatch_tokens_per_rank, num_experts
    L = E // R
    act = [1] * R if active is None else [int(a) for a in active]
    H = next(x.size(1) for x, a in zip(xs, act) if x is not None)
    S = H // 128
    # what every source would send, quantised once per source token
    q, sc, sel = [None] * R, [None] * R, [None] * R
    for r in range(R):
        if not act[r] or xs[r] is None:
            continue
        T = xs[r].size(0)
        assert T <= M
        if use_fp8:
            q[r], sc[r] = fp8_quant(xs[r], arith)
        idx = topks[r].to(torch.int64)
        onehot = torch.zeros((T, E + 1), dtype=torch.bool)
        if T:
            onehot.scatter_(1, torch.where(idx >= 0, idx, torch.full_like(idx, E)), True)
        sel[r] = onehot[:, :E]
    out: List[Optional[dict]] = []
    for r in range(R):
        if not act[r]:
            out.append(None)
            continue
        recv_x = torch.zeros((L, R * M, H), dtype=torch.uint8 if use_fp8 else torch.bfloat16)
        scales = torch.zeros((L, R * M, S), dtype=torch.float32) if use_fp8 else None
        recv_count = torch.zeros((L,), dtype=torch.int32)
        src_info = torch.full((L, R * M), -1, dtype=torch.int32)
        layout_range = torch.zeros((L, R), dtype=torch.int64)
        for le in range(L):
            e = r * L + le
            begin = 0
            for src in range(R):
                if sel[src] is None:
                    continue
                toks = torch.nonzero(sel[src][:, e]).view(-1)
                n = toks.numel()
                if n == 0:
                    continue
                layout_range[le, src] = (begin << 32) | n
                src_info[le, begin:begin + n] = toks.to(torch.int32)
                if use_fp8:
                    recv_x[le, begin:begin + n] = q[src][toks]
                    scales[le, begin:begin + n] = sc[src][toks]
                else:
                    recv_x[le, begin:begin + n] = xs[src][toks]
                begin += n
            recv_count[le] = begin
        out.append(dict(recv_x=recv_x, scales=scales, recv_count=recv_count,
                        src_info=src_info, layout_range=layout_range))
    return out


# --------------------------------------------------------------------------
# combine
# --------------------------------------------------------------------------
def combine(ys: Sequence[Optional[torch.Tensor]],
            topks: Sequence[Optional[torch.Tensor]],
            weights: Sequence[Optional[torch.Tensor]],
            handles: Sequence[Optional[dict]],
            num_max_dispatch_tokens_per_rank: int, num_experts: int,
            active: Optional[Sequence[int]] = None, arith: str = "kernel",
            want_f32: bool = False) -> List[Optional[torch.Tensor]]:
    """All ranks' combine outputs (`[T_r, H]` bf16, or fp32 with `want_f32`).

    `ys[o]` is rank o's expert output `[L, R*M, H]` bf16 in the packed layout
    its dispatch returned; `handles[o]` carries that dispatch's `src_info` and
    `layout_range`. A (token, k) entry contributes when `topk >= 0` and the
    expert's owner is active (mooncake_ep_kernel.cu:728-732).
    """
    R = len(ys)
    M, E = num_max_dispatch_tokens_per_rank, num_experts
    L = E // R
    act = [1] * R if active is None else [int(a) for a in active]
    H = next(y.size(2) for y, a in zip(ys, act) if y is not None and a)
    out: List[Optional[torch.Tensor]] = []
    for r in range(R):
        if not act[r] or topks[r] is None:
            out.append(None)
            continue
        idx = topks[r].to(torch.int64)
        T, K = idx.shape
        # (token, expert) -> packed row on the owner, from the owners' handles
        rowmap = torch.full((T, E), -1, dtype=torch.int64)
        for o in range(R):
            if not act[o] or handles[o] is None:
                continue
            lr, si = handles[o]["layout_range"], handles[o]["src_info"]
            for le in range(L):
                entry = int(lr[le, r])
                begin, n = (entry >> 32) & 0xFFFFFFFF, entry & 0xFFFFFFFF
                if n:
                    toks = si[le, begin:begin + n].to(torch.int64)
                    rowmap[toks, o * L + le] = torch.arange(begin, begin + n)
        gathered = torch.zeros((T * K, H), dtype=torch.bfloat16)
        row_index = torch.full((T, K), -1, dtype=torch.int64)
        for t in range(T):
            for k in range(K):
                e = int(idx[t, k])
                if e < 0 or not act[e // L]:
                    continue
                row = int(rowmap[t, e])
                assert row >= 0, f"rank {r} token {t} expert {e} was never dispatched"
                gathered[t * K + k] = ys[e // L][e % L, row]
                row_index[t, k] = t * K + k
        w = weights[r].to(torch.float32).contiguous()
        if arith == "fallback" and not want_f32:
            # bf16 running sum, each step `bf16(fp32(sum) + fp32(row) * w)`,
            # expert-ascending as the torch path visits them
            # (mooncake_ep_buffer.py:1018-1045); the cross-rank all-reduce then
            # adds the per-owner partials in bf16.
            res = torch.zeros((R, T, H), dtype=torch.bfloat16)
            order = sorted((int(idx[t, k]), t, k) for t in range(T) for k in range(K)
                           if row_index[t, k] >= 0)
            for e, t, k in order:
                res[e // L, t] += gathered[t * K + k] * w[t, k:k + 1]
            out.append(res.sum(dim=0).to(torch.bfloat16) if R > 1 else res[0])
            continue
        if want_f32:
            o32 = torch.empty((T, H), dtype=torch.float32)
            if T:
                lib().ora_combine_reduce_f32(gathered.data_ptr(), row_index.data_ptr(),
                                             w.data_ptr(), T, K, H, o32.data_ptr())
            out.append(o32)
        else:
            o16 = torch.empty((T, H), dtype=torch.bfloat16)
            if T:
                lib().ora_combine_reduce(gathered.data_ptr(), row_index.data_ptr(),
                                         w.data_ptr(), T, K, H, o16.data_ptr())
            out.append(o16)
    return out


# --------------------------------------------------------------------------
# helpers shared by tests and the bench's CPU leg
# --------------------------------------------------------------------------
def canonical_rows(res: dict, le: int) -> Dict[str, torch.Tensor]:
    """Valid rows of one local expert keyed for order-insensitive comparison
    (the reference's own tests compare this way:
    mooncake-wheel/tests/test_mooncake_ep.py:63-80)."""
    n = int(res["recv_count"][le])
    lr = res["layout_range"][le]
    src_rank = torch.full((n,), -1, dtype=torch.int64)
    for s in range(lr.numel()):
        entry = int(lr[s])
        b, c = (entry >> 32) & 0xFFFFFFFF, entry & 0xFFFFFFFF
        src_rank[b:b + c] = s
    key = src_rank * (1 << 32) + res["src_info"][le, :n].to(torch.int64)
    order = torch.argsort(key)
    d = dict(key=key[order], recv_x=res["recv_x"][le, :n][order])
    if res.get("scales") is not None:
        d["scales"] = res["scales"][le, :n][order]
    return d
