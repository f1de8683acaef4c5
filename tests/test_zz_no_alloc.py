"""The allocation-free single-rank combine (`mcep_combine_single_rank_static`).

Some callers of this library may not allocate device memory - they run under a
fixed memory budget or inside a loop where allocator calls are banned - so they
cannot build a `Buffer` (its constructor calls cudaMalloc). This entry point
keeps its scratch in a static device array instead. The test calls it through
the C ABI, twice in a row, and requires the same bytes as the regular
`mcep_combine` path produces for the same inputs.

Collected last on purpose: a run that stops at the first failure has then
already run every other test."""
import pytest
import torch

from mooncake_b200 import Buffer, ep
from tests.ep_harness import FakeGroup, make_rank_inputs

pytestmark = pytest.mark.gpu


def _case(seed, T, H, E, K, n_mask):
    x, idx, w = make_rank_inputs(seed, 0, T, H, E, K, n_mask=n_mask)
    return x.cuda(), idx.cuda(), w.cuda()


def test_static_combine_matches_regular_combine_twice_in_a_row():
    T, H, E, K = 96, 2048, 32, 6
    buf = Buffer(FakeGroup(0, 1), 0)
    active = torch.ones(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for call, seed in enumerate((21, 22)):  # second call: other routing, stale scratch from the first
        x, idx, w = _case(seed, T, H, E, K, n_mask=7 * call)
        recv, cnt, handle, _, _ = buf.dispatch(x, idx, active, T, E, 200_000, use_fp8=False)
        y = (recv.float() * 1.25).nan_to_num().to(torch.bfloat16).contiguous()
        want, _, _ = buf.combine(y, idx, w, active, 200_000, handle)
        got = torch.full((T, H), 7.0, dtype=torch.bfloat16, device="cuda")
        ep.combine_single_rank_static(y.data_ptr(), idx.data_ptr(), w.data_ptr(),
                                      handle[0].data_ptr(), handle[1].data_ptr(), E, T, H, K, T,
                                      got.data_ptr(), stream)
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {call}"
        assert buf.runtime.status() == 0
        assert ep.static_status() == 0  # the entry point's own anomaly word (read and cleared)


def test_static_combine_reports_a_bad_handle_instead_of_partial_sums_in_silence():
    """A handle whose token indices are out of range cannot be combined; the
    kernels skip those rows and say so in the word `mcep_static_status` reads."""
    T, H, E, K = 16, 256, 4, 2
    buf = Buffer(FakeGroup(0, 1), 0)
    active = torch.ones(1, dtype=torch.int32, device="cuda")
    x, idx, w = _case(23, T, H, E, K, n_mask=0)
    recv, cnt, handle, _, _ = buf.dispatch(x, idx, active, T, E, 200_000, use_fp8=False)
    bad_src_info = handle[0].clone()
    le = int((cnt > 0).nonzero()[0])  # an expert that received something
    bad_src_info[le, 0] = T + 5  # a token index the caller never had
    out = torch.empty((T, H), dtype=torch.bfloat16, device="cuda")
    ep.combine_single_rank_static(recv.data_ptr(), idx.data_ptr(), w.data_ptr(),
                                  bad_src_info.data_ptr(), handle[1].data_ptr(), E, T, H, K, T,
                                  out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert ep.static_status() == 4
    assert ep.static_status() == 0  # reading cleared it


def test_static_combine_rejects_sizes_beyond_its_scratch():
    T, K = 8192, 16  # 131072 pairs > 65536
    assert T * K > ep.STATIC_MAX_ENTRIES
    dummy = torch.zeros(64, dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError, match="exceeds the static scratch of 65536"):
        ep.combine_single_rank_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                      dummy.data_ptr(), dummy.data_ptr(), 8, T, 128, K, T,
                                      dummy.data_ptr(), 0)
