"""CUDA-graph capture of the group path ("graph_mode").

A captured launch is replayed with the arguments it was captured with, so the
call's sequence number - which the words ranks exchange carry - cannot be a
launch argument if a captured layer is to be replayed. In graph mode it lives in
device memory. Here two whole layers (dispatch with its hook, a mock expert,
combine with its hook: the two-micro-batch shape of mooncake-ep/src/
mooncake_ep_buffer.cpp:303-305, 330-335) are captured once on a single rank
that takes the group path, and replayed with new inputs; every replay must
match the oracle and move the call counters on. Real groups replay graphs in
tests/test_gpu_multi.py."""
import pytest
import torch

from mooncake_b200 import Buffer
from oracle import ep_oracle as ora
from tests.ep_harness import FakeGroup, make_rank_inputs

pytestmark = pytest.mark.gpu


def _expert(rx, scales, L, H):
    v = rx.view(L, -1, H // 128, 128).to(torch.bfloat16) * scales.unsqueeze(-1).to(torch.bfloat16)
    return (v.view(L, -1, H) * 1.5).to(torch.bfloat16)


@pytest.mark.parametrize("hooked", [True, False])
def test_captured_layers_replay_with_fresh_call_numbers(hooked):
    T, M, H, E, K = 48, 64, 1024, 16, 4
    buf = Buffer(FakeGroup(0, 1), Buffer.get_ep_buffer_size_hint(M, H, 1, E))
    buf.runtime.set_option("force_staged", 1)
    buf.runtime.set_option("graph_mode", 1)
    ar = torch.ones(1, dtype=torch.int32, device="cuda")
    x0, idx0, w0 = make_rank_inputs(40, 0, T, H, E, K)
    x, idx, w = x0.cuda(), idx0.cuda(), w0.cuda()

    def layer():
        (rx, sc), cnt, handle, _, hook = buf.dispatch(x, idx, ar, M, E, 200_000, use_fp8=True,
                                                      return_recv_hook=hooked)
        if hook:
            hook()
        y = _expert(rx, sc, E, H)
        out, _, hook = buf.combine(y, idx, w, ar, 200_000, handle, return_recv_hook=hooked)
        if hook:
            hook()
        return cnt, handle, y, out

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up outside the capture (an even number of layers)
        layer(), layer()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    before = buf.runtime.call_counts()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, capture_error_mode="thread_local"):
        results = [layer(), layer()]
    assert buf.runtime.call_counts() == before  # a capture runs nothing
    for rep in range(3):
        xn, idxn, wn = make_rank_inputs(41 + rep, 0, T, H, E, K, n_mask=rep * 3)
        x.copy_(xn), idx.copy_(idxn), w.copy_(wn)
        g.replay()
        torch.cuda.synchronize()
        want = ora.dispatch([xn], [idxn], M, E, True)[0]
        for cnt, handle, y, out in results:
            assert torch.equal(cnt.cpu(), want["recv_count"])
            assert torch.equal(handle[1].cpu(), want["layout_range"])
            hd = [dict(src_info=handle[0].cpu(), layout_range=handle[1].cpu())]
            ref = ora.combine([y.cpu()], [idxn], [wn], hd, M, E)[0]
            assert torch.equal(out.cpu().view(torch.int16), ref.view(torch.int16)), f"replay {rep}"
        d, c = buf.runtime.call_counts()
        assert (d, c) == (before[0] + 2 * (rep + 1), before[1] + 2 * (rep + 1))
    # eager calls go on from where the replays left the counters
    cnt, handle, y, out = layer()
    torch.cuda.synchronize()
    assert buf.runtime.call_counts() == (before[0] + 7, before[1] + 7)
    assert buf.runtime.status() == 0
