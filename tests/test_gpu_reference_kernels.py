"""A/B against the reference's own CUDA kernels (compiled from a Mooncake
checkout into oracle/_ref/ by oracle/build.py; skipped when that build is
absent). The reference kernel orders an expert's rows by arrival, so both sides
are put into (source rank, token) order before the bytes are compared; then
FP8 payload, scales, counts and the combine output must be identical.

The same file times the reference kernels with the reference's own method
(L2 flush, CUDA events; mooncake-wheel/tests/ep_test_utils.py:79-104) next to
this repository's kernels on the same shape - the "same B200" comparator."""
import ctypes
import json
import os

import pytest
import torch

from mooncake_b200 import Buffer
from tests.ep_harness import FakeGroup, local_group, make_rank_inputs, mock_expert, run_combine, run_dispatch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libmooncake_ep_ref.so")
SEND, RECV = 1, 2
TICKS = 4_000_000_000  # about two seconds of SM clocks: every wait in the reference is bounded


def _ref():
    if not os.path.exists(REF_SO):
        pytest.skip("reference kernels not built (oracle/build.py --ref needs a Mooncake checkout)")
    L = ctypes.CDLL(REF_SO)
    vp, i32, i64, u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_uint64
    L.ref_last_error.restype = ctypes.c_char_p
    L.ref_dispatch.restype = i32
    L.ref_dispatch.argtypes = [vp, vp, vp, vp, i32, vp, vp, vp, vp, vp, vp, vp, vp,
                               i32, i32, i32, i32, i32, i32, i32, i32, i64, i32, u64]
    L.ref_combine.restype = i32
    L.ref_combine.argtypes = [vp, vp, vp, vp, i32, vp, vp, vp, vp, vp, vp, vp,
                              i32, i32, i32, i32, i32, i32, i32, i64, i32, u64]
    return L


class RefGroup:
    """R logical ranks of the reference kernels on one GPU (own buffers, mapped
    to each other through the peer table the kernels take)."""

    def __init__(self, lib, R, M, H, E):
        self.lib, self.R, self.M, self.H, self.E = lib, R, M, H, E
        nbytes = Buffer.get_ep_buffer_size_hint(M, H, R, E)
        self.bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(R)]
        self.ws = [torch.zeros(32 << 20, dtype=torch.uint8, device="cuda") for _ in range(R)]
        self.avail = torch.ones(R, dtype=torch.int32, device="cuda")
        self.peers = torch.tensor([b.data_ptr() for b in self.bufs], dtype=torch.int64, device="cuda")
        self.half = 0

    def _check(self, rc):
        assert rc == 0, self.lib.ref_last_error().decode()

    def dispatch(self, xs, idxs, use_fp8, phases_split, outs=None, sync=True):
        R, M, H, E = self.R, self.M, self.H, self.E
        L = E // R
        half, self.half = self.half, self.half ^ 1
        reuse = outs is not None
        outs = outs if reuse else []
        for r in range(0 if reuse else R):
            o = dict(
                recv_x=torch.empty((L, R * M, H), device="cuda",
                                   dtype=torch.uint8 if use_fp8 else torch.bfloat16),
                scales=torch.empty((L, H // 128, R * M), dtype=torch.float32, device="cuda"),
                src_info=torch.empty((L, R * M), dtype=torch.int32, device="cuda"),
                layout_range=torch.empty((L, R), dtype=torch.int64, device="cuda"),
                recv_count=torch.empty((L,), dtype=torch.int32, device="cuda"),
                active=torch.ones(R, dtype=torch.int32, device="cuda"))
            outs.append(o)
        stream = torch.cuda.current_stream().cuda_stream
        for phases in ((SEND, RECV) if phases_split else (SEND | RECV,)):
            for r in range(R):
                o = outs[r]
                self._check(self.lib.ref_dispatch(
                    self.bufs[r].data_ptr(), self.avail.data_ptr(), self.peers.data_ptr(),
                    self.ws[r].data_ptr(), half, xs[r].data_ptr(), idxs[r].data_ptr(),
                    o["active"].data_ptr(), o["recv_x"].data_ptr(), o["scales"].data_ptr(),
                    o["src_info"].data_ptr(), o["layout_range"].data_ptr(), o["recv_count"].data_ptr(),
                    xs[r].size(0), H, M, idxs[r].size(1), E, r, R, int(use_fp8), TICKS, phases, stream))
        if sync:
            torch.cuda.synchronize()
        return outs

    def combine(self, ys, idxs, ws, outs, phases_split, res=None, sync=True):
        R, M, H, E = self.R, self.M, self.H, self.E
        half, self.half = self.half, self.half ^ 1
        if res is None:
            res = [torch.empty((idxs[r].size(0), H), dtype=torch.bfloat16, device="cuda")
                   for r in range(R)]
        stream = torch.cuda.current_stream().cuda_stream
        for phases in ((SEND, RECV) if phases_split else (SEND | RECV,)):
            for r in range(R):
                o = outs[r]
                self._check(self.lib.ref_combine(
                    self.bufs[r].data_ptr(), self.avail.data_ptr(), self.peers.data_ptr(),
                    self.ws[r].data_ptr(), half, ys[r].data_ptr(), idxs[r].data_ptr(), ws[r].data_ptr(),
                    o["src_info"].data_ptr(), o["layout_range"].data_ptr(), o["active"].data_ptr(),
                    res[r].data_ptr(), idxs[r].size(0), H, M, idxs[r].size(1), E, r, R, TICKS,
                    phases, stream))
        if sync:
            torch.cuda.synchronize()
        return res


def _canonical(recv_x, scales_view, src_info, layout_range, recv_count, le):
    """Valid rows of one expert in (source rank, token) order."""
    n = int(recv_count[le])
    lr = layout_range[le].cpu()
    src_rank = torch.full((n,), -1, dtype=torch.int64)
    for s in range(lr.numel()):
        entry = int(lr[s])
        b, c = (entry >> 32) & 0xFFFFFFFF, entry & 0xFFFFFFFF
        src_rank[b:b + c] = s
    key = src_rank * (1 << 32) + src_info[le, :n].cpu().to(torch.int64)
    order = torch.argsort(key)
    rows = recv_x[le, :n].cpu()[order]
    sc = scales_view[le, :n].cpu()[order] if scales_view is not None else None
    return key[order], rows, sc


CASES = {
    "decode_fp8_r1": dict(R=1, T=128, M=128, H=7168, E=256, K=8, fp8=True),
    "decode_bf16_r1": dict(R=1, T=128, M=128, H=7168, E=256, K=8, fp8=False),
    "c1_fp8_r2": dict(R=2, T=128, M=128, H=2048, E=16, K=4, fp8=True, routing="softmax"),
    "qwen_fp8_zipf_r2": dict(R=2, T=256, M=256, H=4096, E=128, K=8, fp8=True, routing="zipf1.2"),
    "mixtral_bf16_r4": dict(R=4, T=128, M=128, H=4096, E=8, K=2, fp8=False),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_same_bytes_as_the_reference_kernels(name):
    lib = _ref()
    cfg = CASES[name]
    R, M, H, E, K = cfg["R"], cfg["M"], cfg["H"], cfg["E"], cfg["K"]
    L = E // R
    ins = [make_rank_inputs(31, r, cfg["T"], H, E, K, cfg.get("routing", "uniform")) for r in range(R)]
    xs, idxs, ws = [i[0] for i in ins], [i[1] for i in ins], [i[2] for i in ins]
    dx, di, dw = [x.cuda() for x in xs], [i.cuda() for i in idxs], [w.cuda() for w in ws]

    rg = RefGroup(lib, R, M, H, E)
    split = R > 1  # several ranks on one GPU: every send before any receive
    ref = rg.dispatch(dx, di, cfg["fp8"], split)

    bufs = local_group(R, Buffer.get_ep_buffer_size_hint(M, H, R, E), force_staged=True)
    mine = run_dispatch(bufs, xs, idxs, M, E, cfg["fp8"])

    for r in range(R):
        assert torch.equal(mine[r]["recv_count"], ref[r]["recv_count"]), f"rank {r} recv_count"
        my_sc = mine[r]["scales"] if cfg["fp8"] else None
        ref_sc = ref[r]["scales"].transpose(1, 2) if cfg["fp8"] else None
        my_rx = mine[r]["recv_x"].view(torch.uint8) if cfg["fp8"] else mine[r]["recv_x"]
        for le in range(L):
            ka, ra, sa = _canonical(my_rx, my_sc, mine[r]["handle"][0], mine[r]["handle"][1],
                                    mine[r]["recv_count"], le)
            kb, rb, sb = _canonical(ref[r]["recv_x"], ref_sc, ref[r]["src_info"], ref[r]["layout_range"],
                                    ref[r]["recv_count"], le)
            assert torch.equal(ka, kb), f"rank {r} expert {le}: which tokens arrived"
            assert torch.equal(ra.view(torch.uint8), rb.view(torch.uint8)), f"rank {r} expert {le}: payload"
            if cfg["fp8"]:
                assert torch.equal(sa.contiguous().view(torch.int32), sb.contiguous().view(torch.int32)), \
                    f"rank {r} expert {le}: scales"

    # combine: each side gets expert outputs in its own row order, derived from
    # the same function of the (identical) row contents
    def outputs(side, is_ref):
        ys = []
        for r in range(R):
            rx = side[r]["recv_x"]
            if cfg["fp8"]:
                sc = side[r]["scales"].transpose(1, 2) if is_ref else side[r]["scales"]
                deq = (rx.view(torch.uint8).view(torch.float8_e4m3fn).float().view(L, R * M, -1, 128)
                       * sc.unsqueeze(-1)).view(L, R * M, H).to(torch.bfloat16)
            else:
                deq = rx
            ys.append(mock_expert(torch.nan_to_num(deq.float()).to(torch.bfloat16), r, L).contiguous())
        return ys

    ref_out = rg.combine(outputs(ref, True), di, dw, ref, split)
    my_out = run_combine(bufs, outputs(mine, False), idxs, ws, [m["handle"] for m in mine])
    for r in range(R):
        assert torch.equal(my_out[r][0].view(torch.int16), ref_out[r].view(torch.int16)), f"rank {r} combine"


def _bench(fn, warm=10, iters=30):
    flush = torch.empty(256 << 18, dtype=torch.int32, device="cuda")  # 256 MB, as the reference flushes
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        # idle time on the device while the host runs ahead: the Python of the timed
        # call is queued before the GPU reaches the first event
        torch.cuda._sleep(400_000)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b) * 1e3)
    ts.sort()
    return ts[len(ts) // 2]


TIMED_SHAPES = {
    # BASELINE configurations as one rank sees them (all experts local)
    "c1": dict(T=128, H=2048, E=16, K=4, fp8=False, routing="softmax"),
    "c2": dict(T=128, H=7168, E=256, K=8, fp8=True),
    "c3": dict(T=4096, H=7168, E=256, K=8, fp8=False),
    "c4": dict(T=256, H=4096, E=128, K=8, fp8=True, routing="zipf1.2"),
    "c5_t128": dict(T=128, H=4096, E=8, K=2, fp8=False),
    "c5_t4096": dict(T=4096, H=4096, E=8, K=2, fp8=False),
}


@pytest.mark.parametrize("name", sorted(TIMED_SHAPES))
def test_time_reference_kernels_beside_ours_single_gpu(name):
    """Every BASELINE shape on one GPU: median microseconds of dispatch and of
    combine, the reference's kernels (compiled for sm_100a) vs this repository's,
    same inputs, L2 flushed before every call."""
    lib = _ref()
    cfg = TIMED_SHAPES[name]
    T = M = cfg["T"]
    H, E, K, fp8 = cfg["H"], cfg["E"], cfg["K"], cfg["fp8"]
    big = T * K * H > (1 << 27)
    warm, iters = (3, 10) if big else (10, 30)
    x, idx, w = make_rank_inputs(33, 0, T, H, E, K, cfg.get("routing", "uniform"))
    dx, di, dw = x.cuda(), idx.cuda(), w.cuda()
    y = torch.randn((E, M, H), device="cuda").to(torch.bfloat16)
    rg = RefGroup(lib, 1, M, H, E)
    ref = rg.dispatch([dx], [di], fp8, False)
    # the reference side reuses preallocated outputs and never synchronises
    # inside the timed call: only its two launchers are between the events
    res_buf = [torch.empty((T, H), dtype=torch.bfloat16, device="cuda")]
    t_ref_d = _bench(lambda: rg.dispatch([dx], [di], fp8, False, outs=ref, sync=False), warm, iters)
    t_ref_c = _bench(lambda: rg.combine([y], [di], [dw], ref, False, res=res_buf, sync=False), warm, iters)
    del rg, ref
    torch.cuda.empty_cache()

    res = {}
    modes = (("direct", 0),) if big else (("direct", 0), ("group_path", 1))
    for mode, staged in modes:
        buf = Buffer(FakeGroup(0, 1), Buffer.get_ep_buffer_size_hint(M, H, 1, E) if staged else 0)
        buf.runtime.set_option("force_staged", staged)
        ar = torch.ones(1, dtype=torch.int32, device="cuda")
        t_d = _bench(lambda: buf.dispatch(dx, di, ar, M, E, 200_000, use_fp8=fp8), warm, iters)
        # (combine takes the handle of one of the buffer's last two dispatch calls)
        _, _, handle, _, _ = buf.dispatch(dx, di, ar, M, E, 200_000, use_fp8=fp8)
        res[mode] = (t_d, _bench(lambda: buf.combine(y, di, dw, ar, 200_000, handle), warm, iters))
        del buf, handle
        torch.cuda.empty_cache()
    out = dict(shape=f"{name}: {T} tok, hidden {H}, {E} experts, top-{K}, "
                     f"{'fp8' if fp8 else 'bf16'} dispatch, 1 GPU",
               reference_kernel_us=dict(dispatch=t_ref_d, combine=t_ref_c, layer=t_ref_d + t_ref_c),
               ours_us={m: dict(dispatch=v[0], combine=v[1], layer=v[0] + v[1]) for m, v in res.items()},
               note=f"median of {iters}, L2 flushed before each call, CUDA events around the call; "
                    "reference side = its two launchers with preallocated outputs, "
                    "our side = the full Buffer.dispatch/combine call")
    print("REFERENCE_KERNEL_TIMING " + json.dumps(out))
    d = os.environ.get("MCEP_TEST_LOG_DIR", "")
    if os.path.isdir(d):
        path = os.path.join(d, "ref_kernel_timing.json")
        allres = {}
        if os.path.exists(path):
            try:
                allres = json.load(open(path))
                if "shape" in allres:  # a file of the single-shape format
                    allres = {}
            except Exception:
                allres = {}
        allres[name] = out
        with open(path, "w") as f:
            json.dump(allres, f, indent=1)
    assert t_ref_d > 0 and t_ref_c > 0
