"""The checks of the reference's own EP test, re-expressed for this library.

The reference test (mooncake-wheel/tests/test_mooncake_ep.py:27-99) feeds
self-describing payloads - every channel but the last 128 carries a code of the
source rank, the last 128 carry the token index - and then checks, per local
expert: the received count against the gathered routing (:63-64), every row
against its `src_info` and the `layout_range` segment of its source rank
(:66-75), the combine result against the closed form `x * sum(valid weights)`
(:92-94, difference below 1e-5), and that repeating a call gives the same
bytes (:77-80). Here the ranks of a group are logical ranks on one GPU: their
send phases run as one launch, then every rank's receive phase.
"""
from __future__ import annotations

import random

import pytest
import torch

pytestmark = pytest.mark.gpu

from ep_harness import FakeGroup, local_group  # noqa: E402
from mooncake_b200 import Buffer, ep  # noqa: E402

RANK_OFFSET = 128  # codes rank - 128 .. stay exact in bf16 and in e4m3 * scale


def _inputs(rank: int, T: int, H: int, E: int, K: int, seed: int):
    g = torch.Generator().manual_seed(seed + rank)
    x = torch.ones((T, H), dtype=torch.bfloat16) * (rank - RANK_OFFSET)
    x[:, -128:] = torch.arange(T).to(torch.bfloat16).view(-1, 1)
    scores = torch.randn((T, E), generator=g).abs() + 1
    idx = torch.topk(scores, K, dim=-1, largest=True, sorted=True)[1].contiguous()
    w = torch.randn((T, K), generator=g).abs().contiguous()
    rnd = random.Random(seed * 131 + rank)
    for _ in range(10):
        idx[rnd.randint(0, T - 1), rnd.randint(0, K - 1)] = -1
    return x.cuda(), idx.cuda(), w.cuda()


def _cast_back(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    n, h = q.shape
    return (q.float().view(n, -1, 128) * scales.reshape(n, -1, 1)).view(n, h).to(torch.bfloat16)


def _similarity_gap(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double() + 1, b.double() + 1
    return float(1 - 2 * (a * b).sum() / (a * a + b * b).sum())


def _digest(t: torch.Tensor) -> int:
    """Position-weighted sum of the tensor's bytes."""
    if t.numel() == 0:
        return 0
    b = t.reshape(-1).contiguous().view(torch.uint8).to(torch.int64)
    return int((b * (torch.arange(b.numel(), device=b.device) % 8191 + 1)).sum())


def _layer(bufs, xs, idxs, ws, T, E, use_fp8):
    """One dispatch + combine over the whole group; returns per-rank results."""
    R = len(bufs)
    H = xs[0].size(1)
    # the reference test passes a mask of the wrong length (one entry per token);
    # the wrapper then treats every rank as active
    active = torch.ones((T,), dtype=torch.int32, device="cuda")
    pend = []
    for r in range(R):
        pend.append(bufs[r].dispatch(xs[r], idxs[r], active, T, E, -1, use_fp8=use_fp8,
                                     return_recv_hook=True))
    ep.launch_deferred([b.runtime for b in bufs])  # logical ranks: all send phases in one launch
    for p in pend:
        p[4]()
    torch.cuda.synchronize()
    sims = []
    for r in range(R):
        rx = pend[r][0]
        if use_fp8:
            q, s = rx[0], rx[1].contiguous()
            sims.append(_cast_back(q.view(-1, H), s.view(-1, H // 128)).view(q.shape))
        else:
            sims.append(rx.clone())
    cpend = []
    for r in range(R):
        out = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
        cpend.append(bufs[r].combine(sims[r], idxs[r], ws[r], active, -1, pend[r][2],
                                     return_recv_hook=True, out=out))
    for c in cpend:
        c[2]()
    torch.cuda.synchronize()
    return pend, sims, [c[0] for c in cpend]


def _check_layer(R, T, H, E, K, use_fp8, bufs, seed):
    L = E // R
    ins = [_inputs(r, T, H, E, K, seed) for r in range(R)]
    xs, idxs, ws = [i[0] for i in ins], [i[1] for i in ins], [i[2] for i in ins]
    all_idx = torch.stack(idxs)  # what the reference test all-gathers
    digests = []
    for _ in range(2):  # twice: the second pass must reproduce the first, byte for byte
        pend, sims, combined = _layer(bufs, xs, idxs, ws, T, E, use_fp8)
        dig = 0
        for r in range(R):
            rx, cnt, handle = pend[r][0], pend[r][1], pend[r][2]
            for i in range(L):
                e = r * L + i
                n = int(cnt[i])
                lr = handle[1][i]
                assert n == int((lr & 0xFFFFFFFF).sum())
                assert n == int((all_idx == e).sum())
                rows = sims[r][i, :n].float()
                src = handle[0][i, :n]
                lo, hi = rows[:, :-128].amin(dim=-1), rows[:, :-128].amax(dim=-1)
                assert torch.equal(lo, hi)
                assert float((rows[:, -128:] - (src.view(-1, 1) % T).float()).abs().sum()) == 0
                for j in range(R):
                    begin, count = int(lr[j] >> 32), int(lr[j] & 0xFFFFFFFF)
                    assert int((lo == j - RANK_OFFSET).sum()) == int((all_idx[j] == e).sum())
                    assert count == int((all_idx[j] == e).sum())
                    seg = rows[begin:begin + count, :-128]
                    assert float((seg - (j - RANK_OFFSET)).abs().sum()) == 0
                if use_fp8:
                    dig ^= _digest(rx[0][i, :n]) ^ _digest(rx[1][i, :n].contiguous())
                else:
                    dig ^= _digest(rx[i, :n])
            want = xs[r].float() * ws[r].masked_fill(idxs[r] == -1, 0).sum(dim=1).view(-1, 1)
            assert int(torch.isnan(combined[r]).sum()) == 0
            gap = _similarity_gap(want, combined[r].float())
            assert gap < 1e-5, f"rank {r}: {gap=}"
            dig ^= _digest(combined[r])
        digests.append(dig)
    assert digests[0] == digests[1]


@pytest.mark.parametrize("use_fp8", [False, True])
@pytest.mark.parametrize("R,T,H,E,K", [(8, 128, 7168, 288, 8), (2, 64, 2048, 16, 4)])
def test_self_describing_payloads_group(R, T, H, E, K, use_fp8):
    bufs = local_group(R, Buffer.get_ep_buffer_size_hint(T, H, R, E))
    _check_layer(R, T, H, E, K, use_fp8, bufs, seed=1)
    assert all(b.runtime.status() == 0 for b in bufs)


@pytest.mark.parametrize("use_fp8", [False, True])
def test_self_describing_payloads_single_rank(use_fp8):
    T, H, E, K = 128, 7168, 288, 8
    buf = Buffer(FakeGroup(0, 1), Buffer.get_ep_buffer_size_hint(T, H, 1, E))
    _check_layer(1, T, H, E, K, use_fp8, [buf], seed=2)
    assert buf.runtime.status() == 0


def test_pybind_binding_drives_a_layer(tmp_path):
    """The compiled pybind11 binding (mooncake_b200/csrc/ep_py_mcep.cpp) in the
    place of `mooncake._ep`: one dispatch + combine on a single rank through its
    `Buffer.dispatch` / `Buffer.combine`, with the pointer-and-int argument lists
    of mooncake-ep/include/mooncake_ep_buffer.h:116-133, gives the bytes the
    ctypes binding gives."""
    from pybind_build import build_and_import
    m = build_and_import(str(tmp_path))
    T, H, E, K = 64, 2048, 16, 4
    x, idx, w = _inputs(0, T, H, E, K, seed=3)
    stream = torch.cuda.current_stream().cuda_stream
    active = torch.ones(1, dtype=torch.int32, device="cuda")
    ref_buf = Buffer(FakeGroup(0, 1), 0)
    want_rx, want_cnt, want_handle, _, _ = ref_buf.dispatch(x, idx, active, T, E, 200_000, use_fp8=False)
    want_out, _, _ = ref_buf.combine(want_rx, idx, w, active, 200_000, want_handle)

    b = m.Buffer(0, 1, 0)
    assert b.ibgda_disabled() and b.use_fast_path()
    rx = torch.empty((E, T, H), dtype=torch.bfloat16, device="cuda")
    cnt = torch.empty((E,), dtype=torch.int32, device="cuda")
    src_info = torch.empty((E, T), dtype=torch.int32, device="cuda")
    layout_range = torch.empty((E, 1), dtype=torch.int64, device="cuda")
    ev, hook = b.dispatch(x.data_ptr(), idx.data_ptr(), active.data_ptr(), T, H, K, T, E, 200_000, False,
                          rx.data_ptr(), 0, cnt.data_ptr(), src_info.data_ptr(), layout_range.data_ptr(),
                          False, False, stream)
    assert ev is None and hook is None
    out = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    ev, hook = b.combine(rx.data_ptr(), idx.data_ptr(), w.data_ptr(), src_info.data_ptr(),
                         layout_range.data_ptr(), active.data_ptr(), E, T, H, K, T, E, 200_000, False,
                         out.data_ptr(), True, False, stream)
    assert ev is not None and hook is None
    ev.current_stream_wait(stream)
    torch.cuda.synchronize()
    assert torch.equal(cnt, want_cnt) and torch.equal(layout_range, want_handle[1])
    for e in range(E):
        n = int(cnt[e])
        assert torch.equal(rx[e, :n], want_rx[e, :n]) and torch.equal(src_info[e, :n], want_handle[0][e, :n])
    assert torch.equal(out.view(torch.int16), want_out.view(torch.int16))
    with pytest.raises(RuntimeError, match="Failed: Assertion error"):
        b.dispatch(x.data_ptr(), idx.data_ptr(), active.data_ptr(), T, H, K, T, E, 200_000, False,
                   rx.data_ptr(), 0, cnt.data_ptr(), src_info.data_ptr(), layout_range.data_ptr(),
                   True, True, stream)


def test_pybind_elastic_binding_drives_a_layer(tmp_path):
    """`ElasticBuffer` of the compiled binding in the place of `mooncake._ep.ElasticBuffer`:
    a dispatch and a combine on a single rank with the argument lists the reference's
    wrapper passes (mooncake-wheel/mooncake/mooncake_elastic_buffer.py:602-633, 736-756)
    give what the package's own wrapper gives."""
    from pybind_build import build_and_import
    from mooncake_b200 import ElasticBuffer
    m = build_and_import(str(tmp_path))
    T, H, E, K = 48, 1024, 16, 4
    x, idx, w = _inputs(0, T, H, E, K, seed=4)
    stream = torch.cuda.current_stream().cuda_stream
    ref = ElasticBuffer(FakeGroup(0, 1), num_max_tokens_per_rank=T, hidden=H, num_topk=K)
    want_rx, want_idx, want_w, want_h, _ = ref.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E,
                                                        num_max_tokens_per_rank=T, do_cpu_sync=True)
    want_out, _, _ = ref.combine(want_rx.contiguous(), want_h)
    torch.cuda.synchronize()

    b = m.ElasticBuffer(0, 1, 0, T, H, K, False, False, True, True, True, 3, 0, 300, 10)
    assert b.ibgda_disabled() and b.use_fast_path() and b.get_logical_domain_size() == (1, 1)
    active = torch.ones(1, dtype=torch.int32, device="cuda")
    i32 = lambda *s: torch.empty(s, dtype=torch.int32, device="cuda")  # noqa: E731
    psum_rank, psum_expert, slot, md = i32(1), i32(E + 1), i32(T, K), i32(T, K + 2)
    rx = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    ridx = torch.empty((T, K), dtype=torch.int64, device="cuda")
    rw = torch.empty((T, K), dtype=torch.float32, device="cuda")
    ev = b.dispatch(x.data_ptr(), 2, 0, T, H, 0, 0, 0, idx.data_ptr(), K, w.data_ptr(), active.data_ptr(), E, T, 1,
                    24, False, False, stream, False, psum_rank.data_ptr(), psum_expert.data_ptr(),
                    slot.data_ptr(), 0, 0, rx.data_ptr(), 0, ridx.data_ptr(), rw.data_ptr(), md.data_ptr())
    assert ev is None
    out = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    ev = b.combine(rx.data_ptr(), T, H, idx.data_ptr(), T, K, 0, psum_rank.data_ptr(), md.data_ptr(), 0, 0,
                   active.data_ptr(), E, T, False, 24, True, stream, out.data_ptr())
    assert ev is not None
    ev.current_stream_wait(stream)
    torch.cuda.synchronize()
    n = int(psum_rank[-1])
    assert n == want_rx.shape[0]
    assert torch.equal(rx[:n], want_rx) and torch.equal(ridx[:n], want_idx) and torch.equal(rw[:n], want_w)
    assert torch.equal(md[:n, :2], want_h.recv_src_metadata[:, :2])
    assert torch.equal(psum_expert[1:], want_h.psum_num_recv_tokens_per_expert)
    assert torch.equal(slot, want_h.dst_buffer_slot_idx)
    assert torch.equal(out.view(torch.int16), want_out.view(torch.int16))
