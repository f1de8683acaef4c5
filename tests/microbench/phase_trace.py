"""Where the time goes inside the kernels of one decode-shaped layer on one GPU.

Needs a diagnostic build of the library, in which thread 0 of every block
stamps the SM cycle counter at the phase boundaries of the four kernel bodies
(the stamps are compiled out of the normal library):

    MCEP_LIB=/tmp/libmcep_trace.so MCEP_NVCC_FLAGS=-DMCEP_PHASE_TRACE python mooncake_b200/build.py --force
    MCEP_LIB=/tmp/libmcep_trace.so python tests/microbench/phase_trace.py

Prints, per mode (single-rank direct; staged with one launch per call; staged
with two launches per call) and per body, [mean, min, max] microseconds over
the blocks for every step between two stamps:

    dispatch send    s0 entry | s1 routing of the first token known | s2 payload stores issued |
                     s3 before / s4 after the system fence | s5 counters and flags done
    dispatch receive s0 entry | s1 every flag has a verdict | s2 layout done | s3 rows packed
    combine send     s0 entry | s1 layout read and scanned | s2 rows issued | s3 fence returned | s4 done
    combine reduce   s0 entry | s1 first token's rows located / arrived | s2 done
"""
import ctypes, os, sys, json
sys.path.insert(0, os.getcwd())
import numpy as np
import torch
from mooncake_b200 import Buffer, ep
from tests.ep_harness import FakeGroup, make_rank_inputs

lib = ep._lib
lib.mcep_debug_read_phase_trace.restype = ctypes.c_int
lib.mcep_debug_read_phase_trace.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
MHZ = 1965.0  # SM clock of an unthrottled B200; cycle counts are divided by this

def read():
    a = np.zeros((4, 1024, 8), dtype=np.uint64)
    rc = lib.mcep_debug_read_phase_trace(a.ctypes.data, a.nbytes)
    assert rc == 0
    return a.astype(np.int64)

def stats(name, a, body, nblocks, slots, base_body=None, base=None):
    t = a[body, :nblocks]
    out = {}
    for s in range(1, slots):
        d = (t[:, s] - t[:, s - 1]) / MHZ
        out[f"s{s-1}->s{s}"] = [round(float(d.mean()), 2), round(float(d.min()), 2), round(float(d.max()), 2)]
    g = t[:, 7]
    out["entry_skew_us"] = round(float(g.max() - g.min()) / 1000.0, 2)
    if base is not None:
        d = (t[:, 0] - base[:nblocks, 0]) / MHZ
        out["entry_after_prev_body_entry"] = [round(float(d.mean()), 2), round(float(d.min()), 2), round(float(d.max()), 2)]
    print(name, json.dumps(out))
    return t

T, H, E, K = 128, 7168, 256, 8
x, idx, w = make_rank_inputs(1, 0, T, H, E, K)
x, idx, w = x.cuda(), idx.cuda(), w.cuda()
flush = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
for mode in ("direct", "staged_one_kernel", "staged_split"):
    buf = Buffer(FakeGroup(0, 1), Buffer.get_ep_buffer_size_hint(T, H, 1, E))
    if mode != "direct":
        buf.runtime.set_option("force_staged", 1)
    if mode == "staged_split":
        buf.runtime.set_option("one_kernel", 0)
    act = torch.ones(1, dtype=torch.int32, device="cuda")
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    for it in range(6):
        flush.fill_(it)
        ev[0].record()
        (rx, sc), cnt, handle, _, _ = buf.dispatch(x, idx, act, T, E, 200_000, use_fp8=True)
        ev[1].record()
        y = rx.to(torch.bfloat16)
        flush.fill_(it + 1)
        ev[2].record()
        out, _, _ = buf.combine(y, idx, w, act, 200_000, handle)
        ev[3].record()
        torch.cuda.synchronize()
    print("==", mode, "dispatch us", round(ev[0].elapsed_time(ev[1]) * 1000, 1),
          "combine us", round(ev[2].elapsed_time(ev[3]) * 1000, 1), "status", buf.runtime.status())
    a = read()
    nb = 128
    d0 = stats("dispatch_send", a, 0, nb, 3 if mode == "direct" else 6)
    if mode != "direct":
        nbr = nb if mode == "staged_one_kernel" else int((a[1, :, 0] != 0).sum())
        stats("dispatch_recv", a, 1, nbr, 4, base=a[0] if mode == "staged_one_kernel" else None)
        nbs = int((a[2, :, 0] != 0).sum())
        c0 = stats("combine_send", a, 2, nbs, 5)
        nbr2 = int((a[3, :, 0] != 0).sum())
        stats("combine_reduce", a, 3, min(nbr2, nbs) if mode == "staged_one_kernel" else nbr2, 3,
              base=a[2] if mode == "staged_one_kernel" else None)
        # whole-kernel span from the global timer: first entry to last end cannot be had from
        # cycle counters; report per-block total cycles instead
        if mode == "staged_one_kernel":
            tot = (a[1, :nb, 3] - a[0, :nb, 0]) / MHZ
            print("dispatch kernel per-block total us", round(float(tot.mean()), 2), round(float(tot.max()), 2))
            n2 = min(nbr2, nbs)
            tot = (a[3, :n2, 2] - a[2, :n2, 0]) / MHZ
            print("combine kernel per-block total us", round(float(tot.mean()), 2), round(float(tot.max()), 2), "blocks", nbs, nbr2)
    else:
        stats("combine_reduce", a, 3, nb, 3)
    del buf
