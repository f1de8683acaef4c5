"""One rank of a real multi-GPU parity run (one process per GPU, NCCL only for
the bootstrap). Started by tests/test_gpu_multi.py through torch.distributed.run.

Every rank regenerates all ranks' seeded inputs, runs dispatch + combine through
the public `Buffer` API concurrently with its peers, and compares its own
outputs with the CPU oracle (full-size cases: with properties that need no
oracle). Exit code 0 = parity on this rank."""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from mooncake_b200 import Buffer
from oracle import ep_oracle as ora
from tests.ep_harness import make_rank_inputs, mock_expert


def run_case(cfg, group, rank, R, buf_cache):
    M, E, H, K = cfg["M"], cfg["E"], cfg["H"], cfg["K"]
    L = E // R
    tokens = cfg.get("tokens") or [cfg["T"]] * R
    ins = [make_rank_inputs(cfg.get("seed", 1), r, tokens[r], H, E, K,
                            cfg.get("routing", "uniform"), cfg.get("mask", 0)) for r in range(R)]
    xs, idxs, ws = [i[0] for i in ins], [i[1] for i in ins], [i[2] for i in ins]
    active = cfg.get("active") or [1] * R
    nbytes = Buffer.get_ep_buffer_size_hint(M, H, R, E)
    key = nbytes
    if key not in buf_cache:
        buf_cache.clear()
        buf_cache[key] = Buffer(group, nbytes)
        if rank == 0:
            print("symmetric buffer shared through "
                  + ("fabric handles" if buf_cache[key].runtime.uses_fabric_handles() else "CUDA IPC handles"),
                  flush=True)
    buf = buf_cache[key]
    if cfg.get("refresh_members"):
        # membership refresh (Buffer.update_ep_member): every rank re-exports and
        # re-imports the handles together, with nothing in flight
        torch.cuda.synchronize()
        dist.barrier()
        buf.update_ep_member()
        dist.barrier()
    if not active[rank]:
        return  # an inactive rank makes no call
    # the device-side barrier of the group (ranks marked inactive are not waited for)
    ar_dev = torch.tensor(active, dtype=torch.int32, device="cuda")
    for _ in range(2):
        buf.runtime.barrier(torch.cuda.current_stream().cuda_stream, ar_dev.data_ptr())
    torch.cuda.synchronize()
    assert buf.runtime.status() == 0, "barrier timed out"
    buf.recv_in_place = cfg.get("recv_in_place", True)
    x, idx, w = xs[rank].cuda(), idxs[rank].cuda(), ws[rank].cuda()
    ar = torch.tensor(active, dtype=torch.int32, device="cuda")
    if cfg.get("check") == "properties":
        return run_full_size_case(cfg, buf, rank, R, xs, idxs, ws, x, idx, w, ar)
    if cfg.get("graph"):
        return run_graph_case(cfg, buf, rank, R, xs, idxs, ws, x, idx, w, ar)
    want = ora.dispatch(xs, idxs, M, E, cfg["fp8"], active=active)[rank]
    for rep in range(cfg.get("reps", 2)):  # twice: words, tickets and parities are reused
        mode = cfg.get("mode", "sync")
        recv, cnt, handle, ev, hook = buf.dispatch(
            x, idx, ar, M, E, cfg.get("timeout_us", 5_000_000), use_fp8=cfg["fp8"],
            async_finish=(mode == "async"), return_recv_hook=(mode == "hook"))
        if hook:
            hook()
        if mode == "async":
            ev.current_stream_wait()
        torch.cuda.synchronize()
        rx = recv[0].view(torch.uint8) if cfg["fp8"] else recv
        assert torch.equal(cnt.cpu(), want["recv_count"]), "recv_count"
        assert torch.equal(handle[1].cpu(), want["layout_range"]), "layout_range"
        for le in range(L):
            n = int(cnt[le])
            assert torch.equal(handle[0][le, :n].cpu(), want["src_info"][le, :n]), "src_info"
            assert torch.equal(rx[le, :n].cpu().view(torch.uint8),
                               want["recv_x"][le, :n].view(torch.uint8)), "payload"
            if cfg["fp8"]:
                assert torch.equal(recv[1][le, :n].cpu().contiguous().view(torch.int32),
                                   want["scales"][le, :n].contiguous().view(torch.int32)), "scales"
        if cfg["fp8"]:
            deq = ora.fp8_dequant(rx.cpu().view(-1, H),
                                  recv[1].cpu().contiguous().view(-1, H // 128)).view(L, -1, H).cuda()
        else:
            deq = recv
        y = mock_expert(torch.nan_to_num(deq.float()).to(torch.bfloat16), rank, L).contiguous()
        zero_copy = cfg.get("zero_copy", False)
        if zero_copy:
            buf.get_next_combine_buffer(handle).copy_(y)
            y = torch.empty_like(y)  # only its shape is looked at
        out, ev, hook = buf.combine(y, idx, w, ar, cfg.get("timeout_us", 5_000_000), handle,
                                    zero_copy=zero_copy, async_finish=(mode == "async"),
                                    return_recv_hook=(mode == "hook"))
        if hook:
            hook()
        if mode == "async":
            ev.current_stream_wait()
        torch.cuda.synchronize()
        assert ar.cpu().tolist() == active, f"active_ranks changed: {ar.cpu().tolist()}"
        # closed form: expert e multiplies by (1 + e/16); inactive owners contribute nothing
        f = 1.0 + idxs[rank].clamp_min(0).float() / 16.0
        keep = (idxs[rank] >= 0)
        for r2 in range(R):
            if not active[r2]:
                keep &= (idxs[rank] // L) != r2
        src = xs[rank]
        if cfg["fp8"]:
            q, s = ora.fp8_quant(src)
            src = ora.fp8_dequant(q, s)
        ref = src.float() * (ws[rank] * f * keep).sum(dim=1, keepdim=True)
        if ref.numel():
            err = float((out.cpu().float() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
            assert err < 2e-2, f"combine rel err {err}"
        assert buf.runtime.status() == 0, "device status word set"


def run_graph_case(cfg, buf, rank, R, xs, idxs, ws, x, idx, w, ar):
    """Two layers captured in a CUDA graph on every rank ("graph_mode": the call's
    sequence number lives in device memory) and replayed with rescaled inputs.
    With a stale number a rank would take its peers' words of the previous replay
    for the current ones and read rows before they are written."""
    M, E, H = cfg["M"], cfg["E"], cfg["H"]
    L = E // R
    torch.cuda.synchronize()
    dist.barrier()
    buf.runtime.set_option("graph_mode", 1)

    def layer():
        recv, cnt, handle, _, _ = buf.dispatch(x, idx, ar, M, E, 5_000_000, use_fp8=False)
        y = mock_expert(recv, rank, L)
        out, _, _ = buf.combine(y, idx, w, ar, 5_000_000, handle)
        return cnt, out

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer(), layer()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, capture_error_mode="thread_local"):
        results = [layer(), layer()]
    want = ora.dispatch(xs, idxs, M, E, False)[rank]
    f = 1.0 + idxs[rank].clamp_min(0).float() / 16.0
    keep = (idxs[rank] >= 0)
    for rep in range(4):
        scale = float(rep + 1)
        x.copy_((xs[rank].float() * scale).to(torch.bfloat16))
        g.replay()
        torch.cuda.synchronize()
        ref = (xs[rank].float() * scale).to(torch.bfloat16).float() * (ws[rank] * f * keep).sum(dim=1, keepdim=True)
        for cnt, out in results:
            assert torch.equal(cnt.cpu(), want["recv_count"]), "recv_count"
            err = float((out.cpu().float() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
            assert err < 2e-2, f"replay {rep}: combine rel err {err}"
    assert buf.runtime.status() == 0, "device status word set"
    torch.cuda.synchronize()
    dist.barrier()
    buf.runtime.set_option("graph_mode", 0)


def run_full_size_case(cfg, buf, rank, R, xs, idxs, ws, x, idx, w, ar):
    """Sizes the CPU oracle cannot finish in seconds, checked through properties:
    per-expert counts equal a histogram of all ranks' indices, every segment of
    sampled experts holds its source's rows in token order, and combine with an
    identity expert gives x * sum(w) within bf16 rounding."""
    M, E, H = cfg["M"], cfg["E"], cfg["H"]
    L = E // R
    recv, cnt, handle, _, _ = buf.dispatch(x, idx, ar, M, E, cfg.get("timeout_us", 5_000_000),
                                           use_fp8=False)
    torch.cuda.synchronize()
    src_info, layout_range = handle[0], handle[1]
    mine = torch.arange(rank * L, (rank + 1) * L)
    per_src = torch.stack([torch.bincount(i.view(-1), minlength=E)[mine] for i in idxs], dim=1)
    assert torch.equal(cnt.cpu(), per_src.sum(dim=1).to(torch.int32)), "recv_count"
    lr = layout_range.cpu()
    assert torch.equal(lr & 0xFFFFFFFF, per_src), "layout_range counts"
    for le in (0, L // 2, L - 1):
        for src in range(R):
            begin, n = int(lr[le, src] >> 32), int(lr[le, src] & 0xFFFFFFFF)
            toks = src_info[le, begin:begin + n].cpu().long()
            assert bool((toks[1:] > toks[:-1]).all()), "token order"
            assert bool((idxs[src][toks] == rank * L + le).any(dim=1).all()), "src_info"
            assert torch.equal(recv[le, begin:begin + n].cpu(), xs[src][toks]), "payload"
    for zero_copy in (False, True):
        if zero_copy:
            buf.get_next_combine_buffer(handle).copy_(recv)
        out, _, _ = buf.combine(recv, idx, w, ar, cfg.get("timeout_us", 5_000_000), handle,
                                zero_copy=zero_copy)
        torch.cuda.synchronize()
        ref = xs[rank].float() * ws[rank].sum(dim=1, keepdim=True)
        err = float((out.cpu().float() - ref).abs().max() / ref.abs().max())
        assert err < 1e-2, f"combine rel err {err} (zero_copy={zero_copy})"
    assert buf.runtime.status() == 0, "device status word set"


def run_elastic_case(cfg, group, rank, R):
    """`ElasticBuffer` as a model would use it, in the order of the reference's own
    test (mooncake-ep/tests/test_elastic_buffer.py:229-392): a dispatch with CPU
    sync and its combine, a dispatch with the cached handle, an asynchronous one
    without CPU sync, an expanded one - each compared with the CPU oracle."""
    from mooncake_b200.mooncake_elastic_buffer import ElasticBuffer
    from oracle import elastic_oracle as eo
    from tests.test_elastic_oracle import make_input, route_plan
    M, E, H, K, T = cfg["M"], cfg["E"], cfg["H"], cfg["K"], cfg["T"]
    align = cfg.get("alignment", 1)
    if cfg.get("plan"):
        plans = [route_plan(cfg["plan"], r, R, T, K, E) for r in range(R)]
        idxs = [p[0] for p in plans]
        xs = [make_input(r, T, H, 1_000_000) for r in range(R)]
        ws = [torch.ones((T, K)) for _ in range(R)]
    else:
        plans = None
        ins = [make_rank_inputs(cfg.get("seed", 1), r, T, H, E, K, cfg.get("routing", "uniform"), 4)
               for r in range(R)]
        xs, idxs, ws = [i[0] for i in ins], [i[1] for i in ins], [i[2] for i in ins]
    buf = ElasticBuffer(group, num_max_tokens_per_rank=M, hidden=H, num_topk=K, num_gpu_timeout_secs=10)
    x, idx, w = xs[rank].cuda(), idxs[rank].cuda(), ws[rank].cuda()
    eq = lambda a, b: torch.equal(a.cpu().view(torch.int16), b.view(torch.int16))  # noqa: E731

    def check_flat(recv, ridx, rw, handle, want, n, weights=True):
        assert int(handle.psum_num_recv_tokens_per_scaleup_rank[-1]) == want["n"] == n
        assert handle.psum_num_recv_tokens_per_scaleup_rank.cpu().tolist() == want["psum_rank"].tolist()
        assert eq(recv[:n], want["recv_x"])
        assert torch.equal(ridx[:n].cpu(), want["recv_topk_idx"])
        assert torch.equal(handle.recv_src_metadata[:n, :2].cpu(), want["recv_src_metadata"][:, :2])
        assert torch.equal(handle.dst_buffer_slot_idx.cpu(), want["dst_buffer_slot_idx"])
        if weights:
            assert torch.equal(rw[:n].cpu(), want["recv_topk_weights"])

    # 1. CPU-sync dispatch: exact extents, per-expert counts on the host
    want = eo.elastic_dispatch(xs, idxs, ws, E, M, align)
    recv0, idx0, w0, h0, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E,
                                          num_max_tokens_per_rank=M, expert_alignment=align,
                                          do_cpu_sync=True)
    torch.cuda.synchronize()
    n0 = want[rank]["n"]
    assert recv0.shape[0] == n0 and idx0.shape[0] == n0
    check_flat(recv0, idx0, w0, h0, want[rank], n0)
    assert h0.num_recv_tokens_per_expert_list == [(c + align - 1) // align * align
                                                   for c in want[rank]["hits"]]
    assert h0.psum_num_recv_tokens_per_expert.cpu().tolist() == want[rank]["psum_expert"].tolist()[1:]
    if plans:
        assert n0 == plans[rank][1]
    y0 = (recv0.float() * (1.0 + rank / 8.0)).to(torch.bfloat16)
    ys = [(want[r]["recv_x"].float() * (1.0 + r / 8.0)).to(torch.bfloat16) for r in range(R)]
    comb0, _, _ = buf.combine(y0.contiguous(), h0, topk_weights=w0.contiguous())
    torch.cuda.synchronize()
    ref = eo.elastic_combine(ys, want, idxs, E)
    assert eq(comb0, ref[rank])

    # 2. the cached handle, new data, no routing inputs
    xs1 = [(v.float() * 0.5 + 17).to(torch.bfloat16) for v in xs]
    want1 = eo.elastic_dispatch(xs1, idxs, None, E, M, align)
    recv1, idx1, _, h1, _ = buf.dispatch(xs1[rank].cuda(), handle=h0, num_experts=E, num_max_tokens_per_rank=M)
    torch.cuda.synchronize()
    check_flat(recv1, idx1, None, h1, want1[rank], n0, weights=False)
    assert torch.equal(idx1[:n0], idx0[:n0])
    comb1, _, _ = buf.combine(recv1[:max(n0, 1)].contiguous(), h1)
    torch.cuda.synchronize()
    ref1 = eo.elastic_combine([o["recv_x"] for o in want1], want1, idxs, E)
    assert eq(comb1, ref1[rank])
    if plans:
        torch.testing.assert_close(comb1.cpu(), (xs1[rank].float() * plans[rank][2]).to(torch.bfloat16),
                                   rtol=5e-2, atol=1e-3)

    # 3. asynchronous, no CPU sync: outputs keep their capacity, the count is on the device
    recv2, idx2, w2, h2, ev2 = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E,
                                            num_max_tokens_per_rank=M, expert_alignment=align,
                                            do_cpu_sync=False, async_with_compute_stream=True)
    ev2.current_stream_wait()
    torch.cuda.synchronize()
    assert recv2.shape[0] == R * M and not h2.num_recv_tokens_per_expert_list
    check_flat(recv2, idx2, w2, h2, want[rank], n0)
    y2 = (recv2.float() * (1.0 + rank / 8.0)).to(torch.bfloat16)
    comb2, _, ev3 = buf.combine(y2, h2, async_with_compute_stream=True)
    ev3.current_stream_wait()
    torch.cuda.synchronize()
    assert eq(comb2, ref[rank])

    # 4. expanded layout
    wantx = eo.elastic_dispatch(xs, idxs, ws, E, M, align, do_expand=True)
    rx, ix, wx, hx, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E,
                                     num_max_tokens_per_rank=M, expert_alignment=align, do_expand=True,
                                     do_cpu_sync=True)
    torch.cuda.synchronize()
    o = wantx[rank]
    assert int(hx.psum_num_recv_tokens_per_scaleup_rank[-1]) == o["n"]
    assert hx.psum_num_recv_tokens_per_expert.cpu().tolist() == o["psum_expert"].tolist()
    assert rx.shape[0] == o["n_expanded"] == wx.shape[0] and ix.shape[0] == o["n"]
    assert hx.num_recv_tokens_per_expert_list == o["hits"]
    used = o["used"][:rx.shape[0]]
    assert torch.equal(rx.cpu()[used].view(torch.int16), o["recv_x"][:rx.shape[0]][used].view(torch.int16))
    assert torch.equal(wx.cpu()[used], o["recv_topk_weights"][:rx.shape[0]][used])
    assert torch.equal(hx.recv_src_metadata.cpu(), o["recv_src_metadata"])
    yx_all = [(wantx[r]["recv_x"].float() * (1.0 + r / 8.0)).to(torch.bfloat16) for r in range(R)]
    yx = (rx.float() * (1.0 + rank / 8.0)).to(torch.bfloat16)
    if yx.shape[0] == 0:
        yx = torch.zeros((1, H), dtype=torch.bfloat16, device="cuda")
    combx, _, _ = buf.combine(yx.contiguous(), hx)
    torch.cuda.synchronize()
    refx = eo.elastic_combine(yx_all, wantx, idxs, E, do_expand=True)
    assert eq(combx, refx[rank])
    assert buf.runtime.status() == 0
    buf.barrier(with_cpu_sync=True)
    assert buf.runtime.status() == 0
    buf.destroy()


def main():
    cases = json.loads(os.environ["MCEP_TEST_CASES"])
    rank, R = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    group = dist.group.WORLD
    cache = {}
    for name, cfg in cases.items():
        try:
            if cfg.get("elastic"):
                run_elastic_case(cfg, group, rank, R)
            else:
                run_case(cfg, group, rank, R, cache)
        except AssertionError as exc:
            print(f"[rank {rank}] case {name} FAILED: {exc}", flush=True)
            raise
        # ranks leave a case together, on the host, with nothing in flight
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            print(f"case {name} ok", flush=True)
    cache.clear()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
