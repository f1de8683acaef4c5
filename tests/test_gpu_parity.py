"""Parity of the CUDA path (through the C ABI, via the `Buffer` wrapper) with the
CPU oracle on the same seeded inputs. Integer outputs, FP8 bytes and scales are
bit-exact; combine is bit-exact against the oracle's fp32-FMA restatement and
within 1e-2 relative of an fp32 reference (the tolerance the task states).

Groups of more than one rank run as logical ranks on one GPU: kernels of
different ranks that wait for one another go out as ONE cooperative launch
(tests/ep_harness.py), never as separate launches."""
import pytest
import torch

from oracle import ep_oracle as ora
from tests.ep_harness import (FakeGroup, connect_local_group, local_group, make_rank_inputs, mock_expert,
                              run_combine, run_dispatch)
from mooncake_b200 import ep
from mooncake_b200.mooncake_ep_buffer import Buffer

pytestmark = pytest.mark.gpu

COMBINE_REL_TOL = 1e-2  # vs fp32, relative to the largest magnitude of the output


def _inputs(cfg):
    R = cfg["R"]
    tokens = cfg.get("tokens") or [cfg["T"]] * R
    xs, idxs, ws = [], [], []
    for r in range(R):
        x, idx, w = make_rank_inputs(cfg.get("seed", 1), r, tokens[r], cfg["H"], cfg["E"],
                                     cfg["K"], cfg.get("routing", "uniform"), cfg.get("mask", 0))
        if cfg.get("mask_all"):
            idx.fill_(-1)
        if cfg.get("repeats"):
            # the same expert twice in a token's list (no valid router does this):
            # sent once, added once per listing in combine
            idx[::3, -1] = idx[::3, 0]
        xs.append(x), idxs.append(idx), ws.append(w)
    return xs, idxs, ws


def _check_dispatch(cfg, got, want, active):
    R, E = cfg["R"], cfg["E"]
    L = E // R
    for r in range(R):
        if active is not None and not active[r]:
            assert got[r] is None
            continue
        g, w = got[r], want[r]
        cnt = g["recv_count"].cpu()
        assert torch.equal(cnt, w["recv_count"]), f"rank {r} recv_count"
        src_info, layout_range = g["handle"][0].cpu(), g["handle"][1].cpu()
        assert torch.equal(layout_range, w["layout_range"]), f"rank {r} layout_range"
        rx = g["recv_x"].cpu()
        rx = rx.view(torch.uint8) if cfg["fp8"] else rx
        sc = g["scales"].cpu() if cfg["fp8"] else None
        for le in range(L):
            n = int(cnt[le])
            assert torch.equal(src_info[le, :n], w["src_info"][le, :n]), f"rank {r} le {le} src_info"
            assert torch.equal(rx[le, :n].view(torch.uint8), w["recv_x"][le, :n].view(torch.uint8)), \
                f"rank {r} le {le} payload"
            if cfg["fp8"]:
                assert torch.equal(sc[le, :n].contiguous().view(torch.int32),
                                   w["scales"][le, :n].contiguous().view(torch.int32)), \
                    f"rank {r} le {le} scales"
        if cfg["fp8"]:
            # storage is [L][H/128][R*M]; the returned tensor is its transposed view
            assert g["scales"].stride(1) == 1 and g["scales"].stride(2) == R * cfg["M"]


def _expert_outputs(cfg, got, active):
    R, E, H = cfg["R"], cfg["E"], cfg["H"]
    L = E // R
    ys = [None] * R
    for r in range(R):
        if got[r] is None:
            continue
        if cfg["fp8"]:
            q = got[r]["recv_x"].view(torch.uint8).cpu()
            s = got[r]["scales"].cpu().contiguous()
            deq = ora.fp8_dequant(q.view(-1, H), s.view(-1, H // 128)).view(L, -1, H).cuda()
        else:
            deq = got[r]["recv_x"]
        ys[r] = mock_expert(torch.nan_to_num(deq.float()).to(torch.bfloat16), r, L).contiguous()
    return ys


def _run_case(cfg, active=None, force_staged=True, mode="hook", zero_copy=False,
              recv_in_place=True, bufs=None):
    """mode "hook": send and receive phases as launches of their own; "sync": no
    hook, so small batches take the one-launch path."""
    R, M, E, H = cfg["R"], cfg["M"], cfg["E"], cfg["H"]
    xs, idxs, ws = _inputs(cfg)
    nbytes = Buffer.get_ep_buffer_size_hint(M, H, R, E)
    if bufs is None:
        bufs = local_group(R, nbytes, force_staged=force_staged, recv_in_place=recv_in_place)
    got = run_dispatch(bufs, xs, idxs, M, E, cfg["fp8"], active, mode=mode)
    want = ora.dispatch(xs, idxs, M, E, cfg["fp8"], active=active)
    _check_dispatch(cfg, got, want, active)

    ys = _expert_outputs(cfg, got, active)
    handles = [g["handle"] if g is not None else None for g in got]
    res = run_combine(bufs, ys, idxs, ws, handles, active, mode=mode, zero_copy=zero_copy)
    ys_cpu = [y.cpu() if y is not None else None for y in ys]
    hd = [dict(src_info=h[0].cpu(), layout_range=h[1].cpu()) if h is not None else None
          for h in handles]
    want_c = ora.combine(ys_cpu, idxs, ws, hd, M, E, active=active)
    want_f = ora.combine(ys_cpu, idxs, ws, hd, M, E, active=active, want_f32=True)
    for r in range(R):
        if res[r] is None:
            continue
        out = res[r][0].cpu()
        assert torch.equal(out.view(torch.int16), want_c[r].view(torch.int16)), f"rank {r} combine"
        if out.numel():
            ref = want_f[r]
            err = (out.float() - ref).abs().max() / ref.abs().max().clamp_min(1e-30)
            assert float(err) < COMBINE_REL_TOL
    for b in bufs:
        assert b.runtime.status() == 0
    return got, res


CASES = {
    # the CPU-runnable case (2 ranks, hidden 2048, 16 experts, top-4), both payload types
    "c1_bf16": dict(R=2, T=128, M=128, H=2048, E=16, K=4, fp8=False, routing="softmax"),
    "c1_fp8": dict(R=2, T=128, M=128, H=2048, E=16, K=4, fp8=True, routing="softmax"),
    # config 2: DeepSeek-V3-shaped decode, FP8
    "c2_fp8": dict(R=8, T=128, M=128, H=7168, E=256, K=8, fp8=True),
    # config 3, reduced token count (the oracle has to finish in seconds)
    "c3_bf16_small": dict(R=2, T=384, M=384, H=7168, E=256, K=8, fp8=False),
    # config 4: Qwen3-shaped, Zipf(1.2) routing, FP8
    "c4_fp8_zipf": dict(R=8, T=256, M=256, H=4096, E=128, K=8, fp8=True, routing="zipf1.2"),
    # config 5: Mixtral-shaped sweep
    "c5_r2_t1": dict(R=2, T=1, M=1, H=4096, E=8, K=2, fp8=False),
    "c5_r4_t16": dict(R=4, T=16, M=16, H=4096, E=8, K=2, fp8=False),
    "c5_r8_t128": dict(R=8, T=128, M=128, H=4096, E=8, K=2, fp8=False),
    "c5_r2_t1024": dict(R=2, T=1024, M=1024, H=4096, E=8, K=2, fp8=False),
    "c5_r2_t4096": dict(R=2, T=4096, M=4096, H=4096, E=8, K=2, fp8=False),
    # ragged: an empty rank, uneven counts, masked entries, hidden not a multiple of 512
    "ragged_fp8": dict(R=4, tokens=[0, 5, 64, 33], M=64, H=640, E=12, K=3, fp8=True, mask=9),
    "ragged_bf16": dict(R=4, tokens=[7, 0, 64, 1], M=64, H=1152, E=12, K=3, fp8=False, mask=9),
    # one expert per rank, one choice per token
    "k1_l1": dict(R=4, T=32, M=32, H=256, E=4, K=1, fp8=True),
    # a repeated expert inside a token's list
    "repeats_fp8": dict(R=4, T=40, M=40, H=512, E=16, K=4, fp8=True, repeats=True, mask=5),
    # most choices a token may have
    "k16": dict(R=2, T=24, M=24, H=512, E=32, K=16, fp8=True, mask=20),
    # nothing to send at all: no tokens anywhere, and tokens whose every choice is masked
    "all_empty": dict(R=2, tokens=[0, 0], M=8, H=128, E=4, K=2, fp8=True),
    "all_masked": dict(R=2, T=8, M=8, H=128, E=4, K=2, fp8=False, mask_all=True),
    # fewer tokens than the per-rank maximum the buffers are laid out for
    "m_above_t": dict(R=2, T=5, M=32, H=256, E=8, K=2, fp8=True),
    # the largest expert count the library takes (routing layout in its own kernel)
    "experts_4096": dict(R=2, T=64, M=64, H=128, E=4096, K=8, fp8=True),
    # the cases of the real 8-process run (tests/test_gpu_multi.py), as logical ranks
    "r8_c1_bf16": dict(R=8, T=128, M=128, H=2048, E=16, K=4, fp8=False, routing="softmax"),
    "r8_mixtral_t1": dict(R=8, T=1, M=4, H=4096, E=8, K=2, fp8=False),
    "r8_mixtral_t1024": dict(R=8, T=1024, M=1024, H=4096, E=8, K=2, fp8=False),
    "r8_ragged": dict(R=8, tokens=[(7 * r) % 50 for r in range(8)], M=64, H=640, E=64, K=3,
                      fp8=True, mask=6),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_group_matches_oracle(name):
    _run_case(CASES[name])


# small batches without a hook: both phases of a call in ONE launch (the path a
# real group takes for decode-sized batches)
ONE_LAUNCH = ["repeats_fp8", "c1_bf16", "c1_fp8", "c2_fp8", "c4_fp8_zipf", "c5_r2_t1", "c5_r4_t16", "c5_r8_t128",
              "ragged_fp8", "ragged_bf16", "k1_l1", "k16", "all_empty", "all_masked", "m_above_t",
              "r8_mixtral_t1", "r8_ragged"]


@pytest.mark.parametrize("name", ONE_LAUNCH)
def test_group_one_launch_matches_oracle(name):
    _run_case(CASES[name], mode="sync")


@pytest.mark.parametrize("name", ["c2_fp8", "ragged_bf16", "c5_r2_t1024"])
@pytest.mark.parametrize("mode", ["hook", "sync"])
def test_zero_copy_combine_matches_oracle(name, mode):
    """Expert outputs written into `get_next_combine_buffer` and combined with
    zero_copy=True give the same bytes as the copying path."""
    _run_case(CASES[name], mode=mode, zero_copy=True)


@pytest.mark.parametrize("name", ["c2_fp8", "c1_bf16", "ragged_fp8", "c5_r2_t1024"])
def test_caller_owned_recv_x_matches_oracle(name):
    """A binding that passes a tensor of its own as packed_recv_x (as the
    reference's wrapper does) gets the rows copied out into it."""
    _run_case(CASES[name], recv_in_place=False)


def test_two_layers_in_flight_and_repeated_combine():
    """dispatch A, dispatch B, combine A, combine B on one buffer (two
    micro-batches), then combine A again: the tensors and the recorded rows of
    both calls stay valid, and a handle can be combined more than once."""
    cfgA = dict(R=4, T=48, M=64, H=1024, E=16, K=4, fp8=True, seed=11)
    cfgB = dict(R=4, T=64, M=64, H=1024, E=16, K=4, fp8=True, seed=12)
    R, M, E = 4, 64, 16
    bufs = local_group(R, Buffer.get_ep_buffer_size_hint(M, 1024, R, E))
    ins = {n: _inputs(c) for n, c in (("A", cfgA), ("B", cfgB))}
    got = {n: run_dispatch(bufs, ins[n][0], ins[n][1], M, E, True) for n in ("A", "B")}
    for n, c in (("A", cfgA), ("B", cfgB)):
        _check_dispatch(c, got[n], ora.dispatch(ins[n][0], ins[n][1], M, E, True), None)
    for n, c in (("A", cfgA), ("B", cfgB), ("A", cfgA)):
        ys = _expert_outputs(c, got[n], None)
        handles = [g["handle"] for g in got[n]]
        res = run_combine(bufs, ys, ins[n][1], ins[n][2], handles)
        hd = [dict(src_info=h[0].cpu(), layout_range=h[1].cpu()) for h in handles]
        want = ora.combine([y.cpu() for y in ys], ins[n][1], ins[n][2], hd, M, E)
        for r in range(R):
            assert torch.equal(res[r][0].cpu().view(torch.int16), want[r].view(torch.int16)), (n, r)
    # a third dispatch reuses A's memory: A's handle is no longer one of the last two
    run_dispatch(bufs, ins["A"][0], ins["A"][1], M, E, True)
    with pytest.raises(RuntimeError, match="last two dispatch calls"):
        run_combine(bufs, _expert_outputs(cfgB, got["B"], None), ins["B"][1], ins["B"][2],
                    [g["handle"] for g in got["A"]])
    for b in bufs:
        assert b.runtime.status() == 0


SINGLE = {
    "c2_shape_fp8": dict(R=1, T=128, M=128, H=7168, E=256, K=8, fp8=True),
    "c2_shape_bf16": dict(R=1, T=128, M=128, H=7168, E=256, K=8, fp8=False),
    "mixtral_fp8": dict(R=1, T=64, M=64, H=4096, E=8, K=2, fp8=True, mask=5),
    "empty": dict(R=1, T=0, M=8, H=256, E=4, K=2, fp8=True),
    "partial_tile": dict(R=1, T=33, M=40, H=896, E=6, K=3, fp8=True, mask=4),
    # more tokens than SMs: still one launch per call, two blocks per SM
    "t200_fp8": dict(R=1, T=200, M=200, H=1024, E=32, K=4, fp8=True, mask=7),
    "repeats": dict(R=1, T=48, M=48, H=512, E=8, K=4, fp8=False, repeats=True, mask=3),
    "repeats_large": dict(R=1, T=1500, M=1500, H=256, E=32, K=5, fp8=True, repeats=True),
}


@pytest.mark.parametrize("name", sorted(SINGLE))
@pytest.mark.parametrize("staged", [False, True])
def test_single_rank_matches_oracle(name, staged):
    """A single rank writes the packed outputs directly; with `force_staged` it
    goes through symmetric memory and the word exchange like a multi-rank group.
    Same results."""
    _run_case(SINGLE[name], force_staged=staged)


@pytest.mark.parametrize("name", sorted(SINGLE))
@pytest.mark.parametrize("mode", ["sync", "async"])
def test_single_rank_group_path_plain_launches(name, mode):
    """The group path as production launches it (no deferral, no hook): a single
    rank with `force_staged` waits only for words of its own launch, so
    `ep_dispatch` / `ep_combine` - both phases in one launch - run as they do on
    every GPU of a real group. Also through `async_finish`."""
    cfg = SINGLE[name]
    T, M, H, E, K = cfg["T"], cfg["M"], cfg["H"], cfg["E"], cfg["K"]
    xs, idxs, ws = _inputs(cfg)
    buf = Buffer(FakeGroup(0, 1), Buffer.get_ep_buffer_size_hint(M, H, 1, E))
    buf.runtime.set_option("force_staged", 1)
    ar = torch.ones(1, dtype=torch.int32, device="cuda")
    x, idx, w = xs[0].cuda(), idxs[0].cuda(), ws[0].cuda()
    want = ora.dispatch(xs, idxs, M, E, cfg["fp8"])
    kw = dict(async_finish=(mode == "async"))
    small = T * K <= 4096 and T <= 250  # decode-sized: one block per token, one launch per call
    for rep in range(3):  # both parities, and one reuse
        launches = ep.kernel_launch_count()
        rx, cnt, handle, ev, _ = buf.dispatch(x, idx, ar, M, E, 200_000, use_fp8=cfg["fp8"], **kw)
        assert not small or ep.kernel_launch_count() - launches == 1
        if mode == "async":
            ev.current_stream_wait()
        got = [dict(recv_x=rx[0] if cfg["fp8"] else rx, scales=rx[1] if cfg["fp8"] else None,
                    recv_count=cnt, handle=handle, active=ar)]
        torch.cuda.synchronize()
        _check_dispatch(cfg, got, want, None)
        ys = _expert_outputs(cfg, got, None)
        launches = ep.kernel_launch_count()
        out, ev, _ = buf.combine(ys[0], idx, w, ar, 200_000, handle, **kw)
        assert not small or ep.kernel_launch_count() - launches == 1
        if mode == "async":
            ev.current_stream_wait()
        torch.cuda.synchronize()
        hd = [dict(src_info=handle[0].cpu(), layout_range=handle[1].cpu())]
        ref = ora.combine([ys[0].cpu()], idxs, ws, hd, M, E)[0]
        assert torch.equal(out.cpu().view(torch.int16), ref.view(torch.int16))
    assert buf.runtime.status() == 0


def test_async_call_beside_a_busy_compute_stream():
    """`async_finish=True` puts the call on the communication stream while the
    caller's stream is busy with other kernels (here: large matrix products queued
    before and after). No block of the one-launch kernels depends on a block that
    may not be resident yet, except on the control block, which is the first to
    be scheduled; the result equals the oracle, nobody is marked inactive."""
    cfg = SINGLE["c2_shape_fp8"]
    T, M, H, E, K = cfg["T"], cfg["M"], cfg["H"], cfg["E"], cfg["K"]
    xs, idxs, ws = _inputs(cfg)
    buf = Buffer(FakeGroup(0, 1), Buffer.get_ep_buffer_size_hint(M, H, 1, E))
    buf.runtime.set_option("force_staged", 1)
    ar = torch.ones(1, dtype=torch.int32, device="cuda")
    x, idx, w = xs[0].cuda(), idxs[0].cuda(), ws[0].cuda()
    a = torch.randn((4096, 4096), device="cuda", dtype=torch.bfloat16)
    want = ora.dispatch(xs, idxs, M, E, True)
    for _ in range(3):
        for _ in range(4):
            a @ a  # a few hundred microseconds of work that fills every SM
        rx, cnt, handle, ev, _ = buf.dispatch(x, idx, ar, M, E, 1_000_000, use_fp8=True,
                                              async_finish=True)
        for _ in range(4):
            a @ a
        ev.current_stream_wait()
        torch.cuda.synchronize()
        got = [dict(recv_x=rx[0], scales=rx[1], recv_count=cnt, handle=handle, active=ar)]
        _check_dispatch(cfg, got, want, None)
        ys = _expert_outputs(cfg, got, None)
        for _ in range(4):
            a @ a
        out, ev, _ = buf.combine(ys[0], idx, w, ar, 1_000_000, handle, async_finish=True)
        for _ in range(4):
            a @ a
        ev.current_stream_wait()
        torch.cuda.synchronize()
        hd = [dict(src_info=handle[0].cpu(), layout_range=handle[1].cpu())]
        ref = ora.combine([ys[0].cpu()], idxs, ws, hd, M, E)[0]
        assert torch.equal(out.cpu().view(torch.int16), ref.view(torch.int16))
    assert ar.tolist() == [1]
    assert buf.runtime.status() == 0


def test_mask_run_rank5_inactive():
    """Config 5's fault-mask run: rank 5 is marked inactive on every rank and
    makes no call; its tokens are dropped and its experts contribute nothing."""
    cfg = dict(R=8, T=128, M=128, H=4096, E=8, K=2, fp8=False)
    active = [1, 1, 1, 1, 1, 0, 1, 1]
    got, res = _run_case(cfg, active=active)
    for r in range(8):
        if r != 5:
            assert got[r]["active"].tolist() == active
            assert int(got[r]["handle"][1].cpu()[0, 5]) == 0


@pytest.mark.parametrize("mode", ["hook", "sync"])
def test_timeout_marks_silent_rank_inactive(mode):
    """A bounded wait that runs out: rank 1 makes no call, rank 0 waits 20 ms for
    rank 1's counts, then records rank 1 as inactive and goes on with its own
    tokens (mooncake-ep/src/mooncake_ep_kernel.cu:417-429; the reference's fault
    test checks the same, mooncake-ep/tests/test_ep_grid.py:148-158). Both with
    launches of their own per phase and through the one-launch path."""
    cfg = dict(R=2, T=32, M=32, H=1024, E=8, K=2, fp8=True, seed=5)
    xs, idxs, ws = _inputs(cfg)
    bufs = local_group(2, Buffer.get_ep_buffer_size_hint(32, 1024, 2, 8))
    ar = torch.ones(2, dtype=torch.int32, device="cuda")
    hooked = mode == "hook"
    rx, cnt, handle, _, hook = bufs[0].dispatch(xs[0].cuda(), idxs[0].cuda(), ar, 32, 8, 20_000,
                                                use_fp8=True, return_recv_hook=hooked)
    ep.launch_deferred([bufs[0].runtime])
    if hook:
        hook()
    torch.cuda.synchronize()
    assert ar.tolist() == [1, 0]
    want = ora.dispatch(xs, idxs, 32, 8, True, active=[1, 0])[0]
    assert torch.equal(cnt.cpu(), want["recv_count"])
    assert torch.equal(handle[1].cpu(), want["layout_range"])
    for le in range(4):
        n = int(cnt[le])
        assert torch.equal(rx[0][le, :n].view(torch.uint8).cpu(), want["recv_x"][le, :n])
    # combine with the mask as dispatch left it: nothing waits for rank 1, its
    # experts are skipped
    y = mock_expert(torch.zeros_like(rx[0], dtype=torch.bfloat16), 0, 4)
    out, _, hook = bufs[0].combine(y, idxs[0].cuda(), ws[0].cuda(), ar, 20_000, handle,
                                   return_recv_hook=hooked)
    ep.launch_deferred([bufs[0].runtime])
    if hook:
        hook()
    torch.cuda.synchronize()
    assert ar.tolist() == [1, 0]
    assert float(out.float().abs().max()) == 0.0
    assert bufs[0].runtime.status() == 0


@pytest.mark.parametrize("mode", ["hook", "sync"])
def test_rank_silent_before_combine_contributes_nothing(mode):
    """The reference's stale-data case (mooncake-ep/tests/test_ep_grid.py:250-369):
    round 1 completes on both ranks; in round 2 rank 1 dispatches and then makes
    no combine call. Rank 0's combine waits 5 ms, marks rank 1 inactive, and its
    result holds nothing of rank 1's experts - in particular no round-1 rows."""
    cfg = dict(R=2, T=32, M=32, H=1024, E=8, K=2, fp8=False, seed=6)
    R, M, E, L = 2, 32, 8, 4
    xs, idxs, ws = _inputs(cfg)
    bufs = local_group(R, Buffer.get_ep_buffer_size_hint(M, 1024, R, E))
    for rnd in range(3):  # rounds 0 and 1 complete (both parities carry old rows), round 2 does not
        got = run_dispatch(bufs, xs, idxs, M, E, False, mode=mode)
        ys = [mock_expert(g["recv_x"], r, L) for r, g in enumerate(got)]
        handles = [g["handle"] for g in got]
        if rnd < 2:
            run_combine(bufs, ys, idxs, ws, handles, mode=mode)
            continue
        ar = torch.ones(2, dtype=torch.int32, device="cuda")
        out, _, hook = bufs[0].combine(ys[0], idxs[0].cuda(), ws[0].cuda(), ar, 5000, handles[0],
                                       return_recv_hook=(mode == "hook"))
        ep.launch_deferred([bufs[0].runtime])
        if hook:
            hook()
        torch.cuda.synchronize()
        assert ar.tolist() == [1, 0]
        hd = [dict(src_info=h[0].cpu(), layout_range=h[1].cpu()) for h in handles]
        want = ora.combine([y.cpu() for y in ys], idxs, ws, hd, M, E, active=[1, 0])[0]
        assert torch.equal(out.cpu().view(torch.int16), want.view(torch.int16))
    assert bufs[0].runtime.status() == 0


def test_masked_rank_rejoins_after_membership_refresh():
    """A rank that sat out some layers (marked inactive everywhere, it makes no
    call) is back in step after every rank refreshes the membership: the call
    counters are brought to the group's largest, and the next layer with all ranks
    active matches the oracle."""
    cfg = dict(R=4, T=24, M=32, H=512, E=16, K=3, fp8=True, seed=8)
    bufs = local_group(4, Buffer.get_ep_buffer_size_hint(32, 512, 4, 16))
    _run_case(cfg, bufs=bufs)
    for _ in range(3):  # an odd number of layers without rank 2: parities drift apart too
        _run_case(cfg, active=[1, 1, 0, 1], bufs=bufs)
    assert bufs[2].runtime.call_counts() != bufs[0].runtime.call_counts()
    connect_local_group(bufs)  # what Buffer.update_ep_member() does in a real group
    assert len({b.runtime.call_counts() for b in bufs}) == 1
    _run_case(cfg, bufs=bufs)
    _run_case(cfg, bufs=bufs, mode="sync")


def test_idle_rank_keeps_in_step_over_several_layers():
    """One rank has no tokens at all, another routes everything to its own
    experts: neither exchanges payload with some of its peers. Every dispatch
    call still exchanges counts and answers with every rank, so nobody can run
    ahead of a slower peer by more than one call; several layers in a row, in
    both launch modes, end without a timeout and with the oracle's results."""
    R, M, H, E, K = 4, 32, 512, 16, 2
    cfg = dict(R=R, tokens=[0, 32, 24, 32], M=M, H=H, E=E, K=K, fp8=True, seed=13)
    bufs = local_group(R, Buffer.get_ep_buffer_size_hint(M, H, R, E))
    xs, idxs, ws = _inputs(cfg)
    idxs[1] = (idxs[1] % (E // R)) + 1 * (E // R)  # rank 1 keeps its tokens at home
    for layer in range(6):
        mode = "hook" if layer % 3 else "sync"
        got = run_dispatch(bufs, xs, idxs, M, E, True, timeout_us=2_000_000, mode=mode)
        _check_dispatch(cfg, got, ora.dispatch(xs, idxs, M, E, True), None)
        ys = _expert_outputs(cfg, got, None)
        handles = [g["handle"] for g in got]
        res = run_combine(bufs, ys, idxs, ws, handles, timeout_us=2_000_000, mode=mode)
        hd = [dict(src_info=h[0].cpu(), layout_range=h[1].cpu()) for h in handles]
        want = ora.combine([y.cpu() for y in ys], idxs, ws, hd, M, E)
        for r in range(R):
            assert torch.equal(res[r][0].cpu().view(torch.int16), want[r].view(torch.int16))
            assert got[r]["active"].tolist() == [1] * R and res[r][1].tolist() == [1] * R
    for b in bufs:
        assert b.runtime.status() == 0


def test_rank_marked_active_without_a_mapping_is_left_alone():
    """active_ranks says 1 for a rank whose buffer was never mapped (masked out
    when the group connected): the kernels must not touch it. They treat it as
    inactive and raise status bit 8 instead of storing through a null pointer."""
    cfg = dict(R=2, T=16, M=16, H=256, E=4, K=2, fp8=False, seed=9)
    xs, idxs, ws = _inputs(cfg)
    bufs = local_group(2, Buffer.get_ep_buffer_size_hint(16, 256, 2, 4))
    connect_local_group(bufs, available=[1, 0])  # rank 1 masked out at connect time
    ar = torch.ones(2, dtype=torch.int32, device="cuda")  # ... but marked active by the caller
    rx, cnt, handle, _, hook = bufs[0].dispatch(xs[0].cuda(), idxs[0].cuda(), ar, 16, 4, 20_000,
                                                use_fp8=False, return_recv_hook=True)
    ep.launch_deferred([bufs[0].runtime])
    hook()
    torch.cuda.synchronize()
    want = ora.dispatch(xs, idxs, 16, 4, False, active=[1, 0])[0]
    assert torch.equal(cnt.cpu(), want["recv_count"])
    assert bufs[0].runtime.status() == 8


@pytest.mark.parametrize("T,K,E,R", [(128, 8, 256, 8), (4096, 8, 256, 1), (256, 8, 128, 8),
                                     (1, 2, 8, 8), (0, 4, 16, 2), (777, 11, 288, 4),
                                     # batches of 512 tokens and more take the two-pass route
                                     (512, 16, 4096, 2), (5000, 3, 2048, 8), (4096, 2, 8, 8),
                                     (40000, 2, 64, 2)])
def test_routing_layout_kernel(T, K, E, R):
    g = torch.Generator().manual_seed(T + K)
    idx = torch.topk(torch.randn((max(T, 1), E), generator=g), K, dim=-1)[1][:T].contiguous()
    for _ in range(min(T, 17)):
        idx[int(torch.randint(0, T, (1,), generator=g)), int(torch.randint(0, K, (1,), generator=g))] = -1
    if T > 3:
        idx[3, K - 1] = idx[3, 0]  # a repeated expert inside one token
    want = ora.routing_layout(idx, E, R)
    d = idx.cuda()
    count = torch.empty(E, dtype=torch.int32, device="cuda")
    rank_count = torch.empty(R, dtype=torch.int32, device="cuda")
    prefix = torch.empty(E, dtype=torch.int32, device="cuda")
    slot = torch.full((max(T * K, 1),), -7, dtype=torch.int32, device="cuda")
    scratch = torch.zeros(ep.routing_layout_scratch_bytes(), dtype=torch.uint8, device="cuda")
    for _ in range(2):  # the scratch word must come back to zero
        ep.routing_layout(d.data_ptr(), T, K, E, R, count.data_ptr(), rank_count.data_ptr(),
                          prefix.data_ptr(), slot.data_ptr(), scratch.data_ptr(),
                          torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert torch.equal(count.cpu(), want["count"])
        assert torch.equal(rank_count.cpu(), want["rank_count"])
        assert torch.equal(prefix.cpu(), want["expert_prefix"])
        assert torch.equal(slot[: T * K].cpu().view(T, K), want["slot"])


def test_full_size_prefill_round_trip_single_gpu():
    """Config 3 at full size on one GPU (4096 tokens, hidden 7168, 256 experts,
    top-8, bf16), checked through properties that need no oracle: per-expert
    counts equal a histogram of the indices, every packed row equals its source
    row, and combine(identity expert) == x * sum(w) within bf16 rounding."""
    from tests.ep_harness import FakeGroup
    T = M = 4096
    H, E, K = 7168, 256, 8
    x, idx, w = make_rank_inputs(3, 0, T, H, E, K)
    x, idx, w = x.cuda(), idx.cuda(), w.cuda()
    buf = Buffer(FakeGroup(0, 1), 0)
    ar = torch.ones(1, dtype=torch.int32, device="cuda")
    rx, cnt, handle, _, _ = buf.dispatch(x, idx, ar, M, E, 200_000, use_fp8=False)
    torch.cuda.synchronize()
    hist = torch.bincount(idx.view(-1), minlength=E).to(torch.int32)
    assert torch.equal(cnt, hist)
    src_info = handle[0]
    for e in (0, 17, 255):
        n = int(cnt[e])
        assert torch.equal(rx[e, :n], x[src_info[e, :n].long()])
        toks = src_info[e, :n]
        assert bool((toks[1:] > toks[:-1]).all())  # token-ascending
    out, _, _ = buf.combine(rx, idx, w, ar, 200_000, handle)
    torch.cuda.synchronize()
    ref = x.float() * w.sum(dim=1, keepdim=True)
    err = (out.float() - ref).abs().max() / ref.abs().max()
    assert float(err) < COMBINE_REL_TOL
    assert buf.runtime.status() == 0


@pytest.mark.parametrize("mode", ["sync", "async", "hook"])
def test_stream_modes_single_rank(mode):
    """`async_finish` returns an event, `return_recv_hook` a callable, plain mode
    neither (mooncake-ep/src/mooncake_ep_buffer.cpp:316-338)."""
    from tests.ep_harness import FakeGroup
    T, H, E, K = 64, 2048, 16, 4
    x, idx, w = make_rank_inputs(9, 0, T, H, E, K)
    x, idx, w = x.cuda(), idx.cuda(), w.cuda()
    buf = Buffer(FakeGroup(0, 1), Buffer.get_ep_buffer_size_hint(T, H, 1, E))
    ar = torch.ones(1, dtype=torch.int32, device="cuda")
    kw = dict(async_finish=(mode == "async"), return_recv_hook=(mode == "hook"))
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        rx, cnt, handle, ev, hook = buf.dispatch(x, idx, ar, T, E, 200_000, use_fp8=False, **kw)
        assert (ev.event is not None) == (mode == "async")
        assert (hook is not None) == (mode == "hook")
        if hook:
            hook()
        if mode == "async":
            ev.current_stream_wait()
        out, ev, hook = buf.combine(rx, idx, w, ar, 200_000, handle, **kw)
        if hook:
            hook()
        if mode == "async":
            ev.current_stream_wait()
    side.synchronize()
    ref = x.float() * w.sum(dim=1, keepdim=True)
    assert float((out.float() - ref).abs().max() / ref.abs().max()) < COMBINE_REL_TOL


def test_argument_errors_raise_runtime_error():
    from tests.ep_harness import FakeGroup
    buf = Buffer(FakeGroup(0, 1), 1 << 20)
    ar = torch.ones(1, dtype=torch.int32, device="cuda")
    x = torch.zeros((4, 256), dtype=torch.bfloat16, device="cuda")
    idx = torch.zeros((4, 2), dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError, match="Failed: Assertion error"):
        buf.dispatch(x, idx, ar, 4, 8, 1000, async_finish=True, return_recv_hook=True)
    buf.runtime.set_option("force_staged", 1)
    with pytest.raises(RuntimeError, match="num_ep_buffer_bytes"):
        buf.dispatch(x.repeat(1, 64), idx, ar, 1024, 8, 1000, use_fp8=False)
