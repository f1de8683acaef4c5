"""Elastic-style dispatch / combine through the C ABI (`mcep_elastic_dispatch`,
`mcep_elastic_combine`) against the CPU oracle, bit for bit: a single rank, and
in-process groups of logical ranks on one GPU (their calls are prepared and
started as one cooperative launch, like the other group tests)."""
import pytest
import torch

from mooncake_b200 import ep
from oracle import elastic_oracle as eo
from tests.ep_harness import local_group, make_rank_inputs

pytestmark = pytest.mark.gpu


def _group(R, M, H, K, staged):
    if R == 1 and not staged:
        return local_group(1, 0, force_staged=False)
    return local_group(R, ep.elastic_buffer_size_hint(M, H, R, K), force_staged=True)


def _dispatch(bufs, xs, idxs, ws, E, M, alignment, expand, keep):
    """Elastic dispatch on all logical ranks; returns per rank the device tensors."""
    R = len(bufs)
    L = E // R
    outs = []
    for r in range(R):
        T, H = xs[r].shape
        K = idxs[r].shape[1]
        n_cap = R * M
        out_cap = n_cap * K if expand else n_cap
        d = dict(
            x=xs[r].cuda(), idx=idxs[r].cuda(), w=None if ws is None else ws[r].cuda(),
            active=torch.ones(R, dtype=torch.int32, device="cuda"),
            psum_rank=torch.full((R,), -7, dtype=torch.int32, device="cuda"),
            psum_expert=torch.full((L + 1,), -7, dtype=torch.int32, device="cuda"),
            slot=torch.full((T, K), -7, dtype=torch.int32, device="cuda"),
            recv_x=torch.zeros((out_cap, H), dtype=torch.bfloat16, device="cuda"),
            recv_idx=torch.full((n_cap, K), -7, dtype=torch.int64, device="cuda"),
            recv_w=None if ws is None else torch.full((out_cap,) if expand else (n_cap, K), -7.0,
                                                      device="cuda"),
            md=torch.full((n_cap, K + 2), -7, dtype=torch.int32, device="cuda"),
            copied=torch.full((T, K), -7, dtype=torch.int64, device="cuda"))
        ev = bufs[r].runtime.elastic_dispatch(
            d["x"].data_ptr(), 2, 0, T, H, 0, 0, 0, d["idx"].data_ptr(), K,
            0 if ws is None else d["w"].data_ptr(), d["active"].data_ptr(), E, M, alignment, expand,
            False, torch.cuda.current_stream().cuda_stream, False, d["psum_rank"].data_ptr(),
            d["psum_expert"].data_ptr(), d["slot"].data_ptr(), d["recv_x"].data_ptr(), 0,
            d["recv_idx"].data_ptr(), 0 if ws is None else d["recv_w"].data_ptr(), d["md"].data_ptr(),
            200_000, d["copied"].data_ptr())
        assert ev is None
        outs.append(d)
    ep.launch_deferred([b.runtime for b in bufs])
    torch.cuda.synchronize()
    keep.append(outs)
    return outs


def _combine(bufs, ys, outs, E, M, expand):
    R = len(bufs)
    res = []
    for r in range(R):
        d = outs[r]
        T, K = d["idx"].shape
        H = d["x"].shape[1]
        out = torch.full((T, H), 3.0, dtype=torch.bfloat16, device="cuda")
        bufs[r].runtime.elastic_combine(
            ys[r].data_ptr(), ys[r].shape[0], H, d["idx"].data_ptr(), T, K, 0,
            d["psum_rank"].data_ptr(), d["md"].data_ptr(), d["active"].data_ptr(), E, M, expand, False,
            torch.cuda.current_stream().cuda_stream, out.data_ptr(), 200_000)
        res.append(out)
    ep.launch_deferred([b.runtime for b in bufs])
    torch.cuda.synchronize()
    return res


def _check_dispatch(outs, want, expand, with_w, K):
    for r, (d, o) in enumerate(zip(outs, want)):
        n = o["n"]
        assert d["psum_rank"].cpu().tolist() == o["psum_rank"].tolist(), r
        assert d["psum_expert"].cpu().tolist() == o["psum_expert"].tolist(), r
        assert torch.equal(d["slot"].cpu(), o["dst_buffer_slot_idx"]), r
        assert torch.equal(d["copied"], d["idx"]), r
        assert torch.equal(d["recv_idx"][:n].cpu(), o["recv_topk_idx"]), r
        assert torch.equal(d["md"][:n, :2].cpu(), o["recv_src_metadata"][:, :2]), r
        # rows beyond the received ones are left alone
        assert bool((d["md"][n:] == -7).all()) and bool((d["recv_idx"][n:] == -7).all())
        if not expand:
            assert torch.equal(d["recv_x"][:n].cpu().view(torch.int16), o["recv_x"].view(torch.int16)), r
            if with_w:
                assert torch.equal(d["recv_w"][:n].cpu(), o["recv_topk_weights"]), r
            continue
        assert torch.equal(d["md"][:n, 2:].cpu(), o["recv_src_metadata"][:, 2:]), r
        used = o["used"]
        got = d["recv_x"][:used.shape[0]].cpu()
        assert torch.equal(got[used].view(torch.int16), o["recv_x"][used].view(torch.int16)), r
        if with_w:
            assert torch.equal(d["recv_w"][:used.shape[0]].cpu()[used], o["recv_topk_weights"][used]), r


def _expert(rows_bf16: torch.Tensor, rank: int) -> torch.Tensor:
    return (rows_bf16.float() * (1.0 + rank / 8.0)).to(torch.bfloat16)


CASES = [
    # R, T per rank, H, E, K, M, routing, alignment, expand, weights, staged
    (1, [37], 256, 8, 2, 64, "uniform", 1, False, True, False),
    (1, [37], 256, 8, 4, 64, "uniform", 4, True, True, False),
    (1, [16], 128, 4, 2, 16, "uniform", 1, False, False, True),
    (2, [33, 20], 512, 16, 4, 64, "uniform", 1, False, True, True),
    (2, [33, 0], 512, 16, 4, 64, "uniform", 1, False, True, True),
    (2, [64, 64], 256, 16, 8, 64, "zipf1.2", 8, True, True, True),
    (4, [17, 32, 5, 29], 512, 32, 8, 32, "uniform", 1, False, True, True),
    (4, [17, 32, 5, 29], 512, 32, 8, 32, "uniform", 2, True, False, True),
    (4, [128, 128, 128, 128], 1024, 64, 8, 128, "uniform", 1, False, True, True),
    (1, [700], 256, 8, 2, 1024, "uniform", 1, False, True, False),        # several rounds of the block scans
    (1, [700], 256, 8, 4, 1024, "uniform", 2, True, True, False),
    (2, [200, 180], 256, 8, 2, 512, "uniform", 1, False, True, True),
    (2, [9, 9], 128, 2, 1, 16, "uniform", 1, True, True, True),          # K = 1, one expert per rank
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"R{c[0]}_T{max(c[1])}_H{c[2]}_E{c[3]}_K{c[4]}_a{c[7]}"
                         f"{'_expand' if c[8] else ''}{'' if c[9] else '_now'}{'' if c[10] else '_direct'}")
def test_elastic_calls_match_the_oracle(case):
    R, Ts, H, E, K, M, kind, alignment, expand, with_w, staged = case
    ins = [make_rank_inputs(41, r, Ts[r], H, E, K, kind, n_mask=3) for r in range(R)]
    xs, idxs = [i[0] for i in ins], [i[1] for i in ins]
    if Ts[0] > 4:
        idxs[0][2, :] = -1  # a token that goes nowhere
    ws = [i[2] for i in ins] if with_w else None
    bufs = _group(R, M, H, K, staged)
    keep = []
    outs = _dispatch(bufs, xs, idxs, ws, E, M, alignment, expand, keep)
    want = eo.elastic_dispatch(xs, idxs, ws, E, M, alignment, expand)
    _check_dispatch(outs, want, expand, with_w, K)

    # combine: the mock expert scales every row by a factor of its rank
    ys_cpu = [_expert(want[r]["recv_x"], r) for r in range(R)]
    ys = [y.cuda() if y.shape[0] else torch.zeros((1, H), dtype=torch.bfloat16, device="cuda") for y in ys_cpu]
    got = _combine(bufs, ys, outs, E, M, expand)
    ref = eo.elastic_combine(ys_cpu, want, idxs, E, expand)
    for r in range(R):
        assert torch.equal(got[r].cpu().view(torch.int16), ref[r].view(torch.int16)), r

    # the same handle combines again; then a second dispatch with the handle's routing and new data
    got2 = _combine(bufs, ys, outs, E, M, expand)
    for r in range(R):
        assert torch.equal(got2[r], got[r])
    xs2 = [(x.float() * 0.5 + 1.0).to(torch.bfloat16) for x in xs]
    outs2 = _dispatch(bufs, xs2, idxs, ws, E, M, alignment, expand, keep)
    want2 = eo.elastic_dispatch(xs2, idxs, ws, E, M, alignment, expand)
    _check_dispatch(outs2, want2, expand, with_w, K)
    for r in range(R):
        n = want[r]["n"]
        assert torch.equal(outs2[r]["recv_idx"][:n], outs[r]["recv_idx"][:n])
        assert bufs[r].runtime.status() == 0


def test_reference_test_plans_on_logical_ranks():
    """The route plans and closed forms of mooncake-ep/tests/test_elastic_buffer.py
    (all-to-all and local), through the C ABI on four logical ranks."""
    from tests.test_elastic_oracle import make_input, route_plan
    R, E, K, T, H, M = 4, 256, 8, 32, 4096, 128
    for route in ("alltoall", "local"):
        plans = [route_plan(route, r, R, T, K, E) for r in range(R)]
        idxs = [p[0] for p in plans]
        xs = [make_input(r, T, H, 1_000_000) for r in range(R)]
        ws = [torch.ones((T, K)) for _ in range(R)]
        bufs = _group(R, M, H, K, True)
        keep = []
        outs = _dispatch(bufs, xs, idxs, ws, E, M, 1, False, keep)
        base = torch.arange(T * H, dtype=torch.float32).view(T, H)
        for r in range(R):
            n = int(outs[r]["psum_rank"][-1])
            assert n == plans[r][1]
            src = outs[r]["md"][:n, 0].long().cpu()
            want = (base[src % M] + (src // M).view(-1, 1).float() * 1_000_000).to(torch.bfloat16)
            assert torch.equal(outs[r]["recv_x"][:n].cpu(), want)
        ys = [outs[r]["recv_x"][:max(1, int(outs[r]["psum_rank"][-1]))].contiguous() for r in range(R)]
        got = _combine(bufs, ys, outs, E, M, False)
        for r in range(R):
            want = (xs[r].float() * plans[r][2]).to(torch.bfloat16)
            torch.testing.assert_close(got[r].cpu(), want, rtol=5e-2, atol=1e-3)


def test_elastic_argument_errors():
    bufs = _group(2, 32, 256, 4, True)
    x = torch.zeros((8, 256), dtype=torch.bfloat16, device="cuda")
    idx = torch.zeros((8, 4), dtype=torch.int64, device="cuda")
    act = torch.ones(2, dtype=torch.int32, device="cuda")
    i32 = lambda *s: torch.zeros(s, dtype=torch.int32, device="cuda")  # noqa: E731
    md = i32(64, 6)
    args = dict(psum_rank=i32(2), psum_expert=i32(5), slot=i32(8, 4), recv_idx=torch.zeros((64, 4), dtype=torch.int64, device="cuda"))

    def call(E=8, elem=2, M=32):
        return bufs[0].runtime.elastic_dispatch(
            x.data_ptr(), elem, 0, 8, 256, 0, 0, 0, idx.data_ptr(), 4, 0, act.data_ptr(), E, M, 1, False,
            False, 0, False, args["psum_rank"].data_ptr(), args["psum_expert"].data_ptr(),
            args["slot"].data_ptr(), torch.zeros((64, 256), dtype=torch.bfloat16, device="cuda").data_ptr(), 0,
            args["recv_idx"].data_ptr(), 0, md.data_ptr(), 1000)

    with pytest.raises(RuntimeError, match="E % R == 0"):
        call(E=7)
    with pytest.raises(RuntimeError, match="x_element_size == 2"):
        call(elem=1)
    with pytest.raises(RuntimeError, match="elastic layout fits"):
        call(M=4096)
    out = torch.zeros((8, 256), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="last two elastic dispatch calls"):
        bufs[0].runtime.elastic_combine(x.data_ptr(), 8, 256, idx.data_ptr(), 8, 4, 0,
                                        args["psum_rank"].data_ptr(), md.data_ptr(), act.data_ptr(), 8, 32,
                                        False, False, 0, out.data_ptr(), 1000)
    # the first call that goes through fixes where the record areas sit; later calls may need less, not more
    call()
    call(M=16)
    with pytest.raises(RuntimeError, match="no more record space"):
        call(M=64)
    torch.cuda.synchronize()


def test_asynchronous_call_followed_by_one_on_the_callers_stream():
    """An asynchronous dispatch (communication stream) and, without waiting for it,
    a second dispatch on the caller's stream: the calls share scratch, so the
    second must queue behind the first; both must match the oracle."""
    from mooncake_b200 import ElasticBuffer
    from tests.ep_harness import FakeGroup
    T, H, E, K = 96, 1024, 8, 4
    buf = ElasticBuffer(FakeGroup(0, 1), num_max_tokens_per_rank=T, hidden=H, num_topk=K, num_gpu_timeout_secs=2)
    ins = [make_rank_inputs(50 + i, 0, T, H, E, K, "uniform", n_mask=4) for i in range(2)]
    dev = [[t.cuda() for t in i] for i in ins]
    busy = torch.empty(64 << 20, dtype=torch.int32, device="cuda")
    for _ in range(3):
        busy.zero_()  # something ahead of the first call on the caller's stream
    ra, ia, wa, ha, eva = buf.dispatch(dev[0][0], topk_idx=dev[0][1], topk_weights=dev[0][2], num_experts=E,
                                       num_max_tokens_per_rank=T, do_cpu_sync=False,
                                       async_with_compute_stream=True)
    rb, ib, wb, hb, _ = buf.dispatch(dev[1][0], topk_idx=dev[1][1], topk_weights=dev[1][2], num_experts=E,
                                     num_max_tokens_per_rank=T, do_cpu_sync=False)
    eva.current_stream_wait()
    torch.cuda.synchronize()
    for (r, i, w, h), (x, idx, wt) in (((ra, ia, wa, ha), ins[0]), ((rb, ib, wb, hb), ins[1])):
        want = eo.elastic_dispatch([x], [idx], [wt], E, T)[0]
        n = want["n"]
        assert int(h.psum_num_recv_tokens_per_scaleup_rank[-1]) == n
        assert torch.equal(r[:n].cpu().view(torch.int16), want["recv_x"].view(torch.int16))
        assert torch.equal(i[:n].cpu(), want["recv_topk_idx"]) and torch.equal(w[:n].cpu(), want["recv_topk_weights"])
        assert h.psum_num_recv_tokens_per_expert.cpu().tolist() == want["psum_expert"].tolist()[1:]
    oa, _, evc = buf.combine(ra, ha, async_with_compute_stream=True)
    ob, _, _ = buf.combine(rb, hb)
    evc.current_stream_wait()
    torch.cuda.synchronize()
    for o, r, (x, idx, wt) in ((oa, ra, ins[0]), (ob, rb, ins[1])):
        want = eo.elastic_dispatch([x], [idx], [wt], E, T)
        ref = eo.elastic_combine([want[0]["recv_x"]], want, [idx], E)[0]
        assert torch.equal(o.cpu().view(torch.int16), ref.view(torch.int16))
    assert buf.runtime.status() == 0


def test_buffer_of_an_odd_size_keeps_the_records_aligned():
    """A buffer a few bytes larger than the hint (not a multiple of 16): the record
    areas are placed from the rounded-down end, the calls work as usual."""
    R, T, H, E, K, M = 2, 24, 256, 8, 4, 32
    bufs = local_group(R, ep.elastic_buffer_size_hint(M, H, R, K) + 13, force_staged=True)
    ins = [make_rank_inputs(61, r, T, H, E, K, "uniform", n_mask=2) for r in range(R)]
    xs, idxs, ws = [i[0] for i in ins], [i[1] for i in ins], [i[2] for i in ins]
    keep = []
    outs = _dispatch(bufs, xs, idxs, ws, E, M, 1, False, keep)
    _check_dispatch(outs, eo.elastic_dispatch(xs, idxs, ws, E, M), False, True, K)
    assert all(b.runtime.status() == 0 for b in bufs)
