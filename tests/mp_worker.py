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


def main():
    cases = json.loads(os.environ["MCEP_TEST_CASES"])
    rank, R = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    group = dist.group.WORLD
    cache = {}
    for name, cfg in cases.items():
        try:
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
