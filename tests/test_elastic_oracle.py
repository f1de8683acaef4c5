"""The elastic oracle against the closed forms the reference's own test checks
(mooncake-ep/tests/test_elastic_buffer.py: route plans :107-152, payload against
metadata :165-198, combine = x * ranks reached :281-283, cached-handle top-k
:323-324, expanded extents :383-392), re-expressed for one process."""
import pytest
import torch

from oracle import elastic_oracle as eo


def route_plan(route: str, rank: int, R: int, T: int, K: int, E: int):
    """The three generators of the reference's test for a single NVLink domain."""
    L = E // R
    offs = torch.arange(K, dtype=torch.long) % L
    if route in ("local", "cross"):  # "cross" needs two domains; with one it is "local" (:138)
        return (rank * L + offs).view(1, K).repeat(T, 1).contiguous(), T, 1
    dst = (rank + torch.arange(K, dtype=torch.long)) % R
    uniq = int(torch.unique(dst).numel())
    return (dst * L + offs).view(1, K).repeat(T, 1).contiguous(), T * uniq, uniq


def make_input(rank: int, T: int, H: int, mult: int, addend: int = 0) -> torch.Tensor:
    base = torch.arange(T * H, dtype=torch.float32).view(T, H)
    return (base + rank * mult + addend).to(torch.bfloat16).contiguous()


@pytest.mark.parametrize("route", ["alltoall", "local", "cross"])
@pytest.mark.parametrize("R,E,K", [(2, 16, 4), (4, 32, 8), (8, 256, 8), (1, 8, 2)])
def test_closed_forms_of_the_reference_test(route, R, E, K):
    T, H, M = 12, 64, 16
    plans = [route_plan(route, r, R, T, K, E) for r in range(R)]
    idxs = [p[0] for p in plans]
    xs = [make_input(r, T, H, 1_000_000) for r in range(R)]
    ws = [torch.ones((T, K)) for _ in range(R)]
    outs = eo.elastic_dispatch(xs, idxs, ws, E, M)
    base = torch.arange(T * H, dtype=torch.float32).view(T, H)
    for r in range(R):
        o = outs[r]
        # every rank receives what the plan of the senders says (symmetric plans)
        assert int(o["psum_rank"][-1]) == plans[r][1] == o["n"]
        src = o["recv_src_metadata"][:, 0].long()
        src_rank, src_tok = src // M, src % M
        assert bool((src_tok < T).all())
        want = (base[src_tok] + src_rank.view(-1, 1).float() * 1_000_000).to(torch.bfloat16)
        assert torch.equal(o["recv_x"], want)
        assert len(o["hits"]) == E // R
        assert int(o["psum_expert"][-1]) == sum(o["hits"])
    comb = eo.elastic_combine([o["recv_x"] for o in outs], outs, idxs, E)
    for r in range(R):
        want = (xs[r].float() * plans[r][2]).to(torch.bfloat16)
        torch.testing.assert_close(comb[r], want, rtol=5e-2, atol=1e-3)
    # a second dispatch with the same routing returns the same top-k metadata
    x1 = [make_input(r, T, H, 2_000_000, 17) for r in range(R)]
    again = eo.elastic_dispatch(x1, idxs, None, E, M)
    for r in range(R):
        assert torch.equal(again[r]["recv_topk_idx"], outs[r]["recv_topk_idx"])
    # expanded layout: extents
    exp = eo.elastic_dispatch(xs, idxs, ws, E, M, do_expand=True)
    for r in range(R):
        assert int(exp[r]["psum_rank"][-1]) == plans[r][1]
        assert exp[r]["recv_x"].shape[0] == int(exp[r]["psum_expert"][-1]) == exp[r]["n_expanded"]


def test_lane_of_a_rank_is_its_last_listing_and_order_follows_lanes():
    R, E, K, M, H = 4, 8, 4, 4, 32  # L = 2
    idx = torch.tensor([[6, 0, 1, 7],     # rank 3 (lanes 0, 3 -> 3), rank 0 (lanes 1, 2 -> 2)
                        [2, -1, 3, 2]])   # rank 1 (lanes 0, 2, 3 -> 3)
    assert eo.rank_lanes(idx[0], 2, E) == {3: 3, 0: 2}
    assert eo.rank_lanes(idx[1], 2, E) == {1: 3}
    xs = [torch.randn((2, H)).to(torch.bfloat16)] + [torch.zeros((0, H), dtype=torch.bfloat16)] * 3
    idxs = [idx] + [torch.zeros((0, K), dtype=torch.int64)] * 3
    outs = eo.elastic_dispatch(xs, idxs, None, E, M)
    slot = outs[0]["dst_buffer_slot_idx"]
    assert slot.tolist() == [[-1, -1, 0, 0], [-1, -1, -1, 0]]
    assert outs[0]["n"] == 1 and outs[1]["n"] == 1 and outs[2]["n"] == 0 and outs[3]["n"] == 1
    assert outs[0]["recv_topk_idx"].tolist() == [[-1, 0, 1, -1]]
    assert outs[0]["recv_src_metadata"][0, :2].tolist() == [0, 0 * K + 2]
    assert outs[3]["recv_topk_idx"].tolist() == [[0, -1, -1, 1]]
    assert outs[3]["recv_src_metadata"][0, :2].tolist() == [0, 3]
    assert outs[0]["psum_expert"].tolist() == [0, 1, 2]


def test_expert_alignment_and_expanded_rows():
    R, E, K, M, H = 2, 4, 2, 8, 32  # L = 2
    g = torch.Generator().manual_seed(5)
    idxs = [torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(6)]) for _ in range(R)]
    xs = [torch.randn((6, H), generator=g).to(torch.bfloat16) for _ in range(R)]
    ws = [torch.rand((6, K), generator=g) for _ in range(R)]
    outs = eo.elastic_dispatch(xs, idxs, ws, E, M, expert_alignment=4, do_expand=True)
    for d in range(R):
        o = outs[d]
        hits = o["hits"]
        start1 = (hits[0] + 3) // 4 * 4
        assert o["psum_expert"].tolist() == [hits[0], start1 + hits[1], start1 + (hits[1] + 3) // 4 * 4]
        md = o["recv_src_metadata"]
        for i in range(o["n"]):
            for k in range(K):
                le = int(o["recv_topk_idx"][i, k])
                row = int(md[i, 2 + k])
                assert (row >= 0) == (le >= 0)
                if le >= 0:
                    assert torch.equal(o["recv_x"][row], o["flat"][i])
                    assert float(o["recv_topk_weights"][row]) == float(ws[int(md[i, 0]) // M][int(md[i, 0]) % M, k])
    # combine of the expanded rows = combine of the per-token sums
    ys = [o["recv_x"] for o in outs]
    comb = eo.elastic_combine(ys, outs, idxs, E, do_expand=True)
    for s in range(R):
        for t in range(6):
            per_rank = {}
            for k, e in enumerate(idxs[s][t].tolist()):
                per_rank.setdefault(e // 2, []).append(xs[s][t])
            lanes = eo.rank_lanes(idxs[s][t], 2, E)
            order = [d for d, _ in sorted(lanes.items(), key=lambda kv: kv[1])]
            rows = [eo.bf16_sum(per_rank[d]) if len(per_rank[d]) > 1 else per_rank[d][0] for d in order]
            assert torch.equal(comb[s][t], eo.bf16_sum(rows))


def test_three_and_more_rows_accumulate_in_fp32_from_zero():
    a = torch.tensor([[1.0, -0.0]], dtype=torch.bfloat16)
    b = torch.tensor([[2.0 ** -9, -0.0]], dtype=torch.bfloat16)
    two = eo.bf16_sum([a[0], b[0]])
    assert two[1].item() == 0.0 and torch.signbit(two[1])        # (-0) + (-0) = -0
    three = eo.bf16_sum([a[0], b[0], b[0]])
    assert not torch.signbit(three[1])                            # 0 + (-0) + ... = +0
    assert three[0].item() == float((torch.tensor(1.0) + 2.0 ** -8).to(torch.bfloat16))
