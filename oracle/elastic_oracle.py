"""CPU oracle for the elastic-style `ElasticBuffer.dispatch` / `.combine`.

TEST INFRASTRUCTURE ONLY: imported by `tests/` alone. The product package never
imports it and has no CPU fallback.

It restates, for all ranks of one NVLink domain at once and in one process, what
the reference's elastic kernels compute (paths relative to the Mooncake tree,
all under mooncake-ep/include/elastic/):

* a token goes once to every rank that owns at least one of its experts; the
  lane that stands for a rank is the LAST lane of the top-k list that names one
  of its experts (`deduplicate` = highest lane of the match group,
  mooncake_ep_elastic_ptx.cuh:679-693; dispatch_official.cuh:113-117,422-436);
* positions inside a destination's per-source region follow the token order
  (the reference's `deterministic` prologue,
  mooncake_ep_elastic_dispatch_deterministic_prologue.cuh:134-166; its default
  mode hands them out atomically, any order);
* the receiver's rows are the sources' regions one after another, source rank
  ascending (dispatch_copy_epilogue.cuh:79-97), with
  `psum_num_recv_tokens_per_scaleup_rank` the inclusive sum of their sizes and
  `psum_num_recv_tokens_per_expert` the exclusive sum of the per-expert hit
  counts rounded up to `expert_alignment` (dispatch_official.cuh:255-310);
* per row: local expert index or -1 per lane, the source's weights, and the
  metadata `[src_rank * M + token, src_rank * K + last lane with a local
  expert, (expand) row of every lane]` (dispatch_copy_epilogue.cuh:114-132,
  212-248);
* expanded layout: one row per (received token, local expert), expert segments
  starting at the aligned exclusive sums; inside an expert this oracle uses the
  receive order (the reference: arrival order of an atomic, :138-141), and the
  per-expert entries of the prefix sum end as the ENDS of the segments;
* combine: with an expanded layout the rows of one received token are first
  summed (one: copied; two: one bf16 addition; more: fp32 from zero, one
  rounding - combine_official.cuh:146-216, combine_utils.cuh:66-205), then one
  row per received token returns to the token's owner, which adds the rows of
  the ranks it reached in the order of their lanes with the same three cases
  (combine_reduce_epilogue.cuh:100-161). No weights enter the sum.

Parity status: parity unpinned. The reference holds no golden vectors for this
interface and its kernels are shape-locked templates over a transport that is
absent here; the oracle is checked against the closed forms of the reference's
own test (mooncake-ep/tests/test_elastic_buffer.py: received-row counts, payload
against metadata, combine = x * number of ranks reached, cached-handle top-k
equality, expanded extents) in tests/test_elastic_oracle.py.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch


def _align(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def rank_lanes(idx_row: torch.Tensor, L: int, E: int) -> Dict[int, int]:
    """rank -> the lane that stands for it (the last one naming one of its experts)."""
    out: Dict[int, int] = {}
    for k, e in enumerate(idx_row.tolist()):
        if 0 <= e < E:
            out[e // L] = k
    return out


def bf16_sum(rows: List[torch.Tensor]) -> torch.Tensor:
    """The reference's reduction of up to K bf16 rows (combine_utils.cuh:66-205)."""
    if len(rows) == 0:
        raise ValueError("nothing to add")
    if len(rows) <= 2:
        # bf16 addition of two rows (a missing second row reads as +0): the exact sum
        # rounded once, which the fp32 sum rounded to bf16 also gives
        a = rows[0].float()
        b = rows[1].float() if len(rows) == 2 else torch.zeros_like(a)
        return (a + b).to(torch.bfloat16)
    acc = torch.zeros_like(rows[0], dtype=torch.float32)
    for r in rows:
        acc = acc + r.float()
    return acc.to(torch.bfloat16)


def elastic_dispatch(xs: List[torch.Tensor], idxs: List[torch.Tensor],
                     ws: Optional[List[torch.Tensor]], num_experts: int, M: int,
                     expert_alignment: int = 1, do_expand: bool = False) -> List[dict]:
    """All ranks' dispatch outputs. xs[r]: [T_r, H] bf16, idxs[r]: [T_r, K] int64."""
    R, E = len(xs), num_experts
    L, K, H = E // R, idxs[0].shape[1], xs[0].shape[1]
    lanes = [[rank_lanes(idxs[s][t], L, E) for t in range(idxs[s].shape[0])] for s in range(R)]
    outs = []
    for s in range(R):  # sender-side tensor
        T = idxs[s].shape[0]
        slot = torch.full((T, K), -1, dtype=torch.int32)
        seen = [0] * R
        for t in range(T):
            for d, k in sorted(lanes[s][t].items()):
                slot[t, k] = s * M + seen[d]
                seen[d] += 1
        outs.append({"dst_buffer_slot_idx": slot})
    for d in range(R):
        rows = [(s, t) for s in range(R) for t in range(idxs[s].shape[0]) if d in lanes[s][t]]
        n = len(rows)
        per_src = [sum(1 for (s, _) in rows if s == q) for q in range(R)]
        psum_rank = torch.tensor(per_src, dtype=torch.int32).cumsum(0).to(torch.int32)
        recv_idx = torch.full((n, K), -1, dtype=torch.int64)
        recv_w = torch.zeros((n, K), dtype=torch.float32)
        md = torch.full((n, K + 2), -1, dtype=torch.int32)
        flat = torch.empty((n, H), dtype=torch.bfloat16)
        hits = [0] * L
        for i, (s, t) in enumerate(rows):
            flat[i] = xs[s][t]
            master = 0
            for k, e in enumerate(idxs[s][t].tolist()):
                if d * L <= e < (d + 1) * L:
                    recv_idx[i, k] = e - d * L
                    hits[e - d * L] += 1
                    master = k
            if ws is not None:
                recv_w[i] = ws[s][t]
            md[i, 0] = s * M + t
            md[i, 1] = s * K + master
        starts = [0]
        for c in hits:
            starts.append(starts[-1] + _align(c, expert_alignment))
        o = outs[d]
        o.update(n=n, psum_rank=psum_rank, recv_topk_idx=recv_idx, recv_src_metadata=md,
                 psum_expert=torch.tensor(starts, dtype=torch.int32), hits=hits, rows=rows)
        if not do_expand:
            o.update(recv_x=flat, recv_topk_weights=recv_w if ws is not None else None)
            continue
        total = starts[L - 1] + hits[L - 1] if L else 0
        ex = torch.zeros((starts[L], H), dtype=torch.bfloat16)
        ew = torch.zeros((starts[L],), dtype=torch.float32)
        used = torch.zeros((starts[L],), dtype=torch.bool)
        fill = list(starts[:L])
        for i in range(n):
            for k in range(K):
                le = int(recv_idx[i, k])
                if le >= 0:
                    ex[fill[le]] = flat[i]
                    ew[fill[le]] = recv_w[i, k]
                    used[fill[le]] = True
                    md[i, 2 + k] = fill[le]
                    fill[le] += 1
        ends = torch.tensor(fill + [starts[L]], dtype=torch.int32)
        o.update(recv_x=ex, recv_topk_weights=ew if ws is not None else None, psum_expert=ends,
                 n_expanded=total, used=used, flat=flat)
    return outs


def elastic_combine(ys: List[torch.Tensor], outs: List[dict], idxs: List[torch.Tensor],
                    num_experts: int, do_expand: bool = False) -> List[torch.Tensor]:
    """ys[d]: what rank d's experts made of its received rows - [n_d, H] bf16, or
    the expanded rows with `do_expand`. Returns every rank's combined [T_r, H]."""
    R, E = len(ys), num_experts
    L, K = E // R, idxs[0].shape[1]
    H = ys[0].shape[1]
    back: List[Dict[tuple, torch.Tensor]] = []
    for d in range(R):
        o = outs[d]
        sent: Dict[tuple, torch.Tensor] = {}
        for i, (s, t) in enumerate(o["rows"]):
            if do_expand:
                slots = [int(v) for v in o["recv_src_metadata"][i, 2:].tolist() if v >= 0]
                row = ys[d][slots[0]].clone() if len(slots) == 1 else bf16_sum([ys[d][j] for j in slots])
            else:
                row = ys[d][i]
            sent[(s, t)] = row
        back.append(sent)
    res = []
    for s in range(R):
        T = idxs[s].shape[0]
        out = torch.zeros((T, H), dtype=torch.bfloat16)
        for t in range(T):
            lanes = rank_lanes(idxs[s][t], L, E)
            order = [d for d, _ in sorted(lanes.items(), key=lambda kv: kv[1])]
            if order:
                out[t] = bf16_sum([back[d][(s, t)] for d in order])
        res.append(out)
    return res
