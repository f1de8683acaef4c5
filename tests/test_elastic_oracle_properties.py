"""Size-independent properties of the elastic oracle on seeded random routing:
what must hold whatever the order conventions are (conservation of rows, the
prefix sums, the slot indices, closed forms of the combine)."""
import pytest
import torch

from oracle import elastic_oracle as eo
from tests.ep_harness import make_rank_inputs

CASES = [  # R, T per rank, H, E, K, M, routing, alignment
    (1, [40], 64, 8, 4, 64, "uniform", 1),
    (2, [31, 17], 64, 16, 4, 32, "uniform", 1),
    (4, [20, 0, 33, 7], 32, 32, 8, 48, "zipf1.2", 4),
    (8, [16] * 8, 32, 64, 8, 16, "uniform", 2),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"R{c[0]}_E{c[3]}_K{c[4]}_a{c[7]}")
def test_rows_prefix_sums_and_slots(case):
    R, Ts, H, E, K, M, kind, align = case
    L = E // R
    ins = [make_rank_inputs(77, r, Ts[r], H, E, K, kind, n_mask=5) for r in range(R)]
    xs, idxs, ws = [i[0] for i in ins], [i[1] for i in ins], [i[2] for i in ins]
    outs = eo.elastic_dispatch(xs, idxs, ws, E, M, align)
    for d in range(R):
        o = outs[d]
        # conservation: exactly the (source, token) pairs that name an expert of d, once each
        want = {(s, t) for s in range(R) for t in range(Ts[s])
                if any(d * L <= e < (d + 1) * L for e in idxs[s][t].tolist())}
        got = [(int(v) // M, int(v) % M) for v in o["recv_src_metadata"][:, 0].tolist()]
        assert len(got) == len(set(got)) == o["n"] and set(got) == want
        assert got == sorted(got)  # source rank, then token
        # payload and per-lane choices of every row
        for i, (s, t) in enumerate(got):
            assert torch.equal(o["recv_x"][i], xs[s][t])
            lanes = [e - d * L if d * L <= e < (d + 1) * L else -1 for e in idxs[s][t].tolist()]
            assert o["recv_topk_idx"][i].tolist() == lanes
            assert torch.equal(o["recv_topk_weights"][i], ws[s][t])
            assert int(o["recv_src_metadata"][i, 1]) == s * K + max(k for k, v in enumerate(lanes) if v >= 0)
        # prefix sums
        per_src = [sum(1 for (s, _) in got if s == q) for q in range(R)]
        assert o["psum_rank"].tolist() == [sum(per_src[:q + 1]) for q in range(R)]
        hits = [sum(int((o["recv_topk_idx"] == le).sum()) for _ in [0]) for le in range(L)]
        assert hits == o["hits"]
        ps = o["psum_expert"].tolist()
        assert ps[0] == 0 and all(ps[j + 1] - ps[j] == (hits[j] + align - 1) // align * align for j in range(L))
    # the sender's slot indices name the row's position inside the sender's segment
    for s in range(R):
        slot = outs[s]["dst_buffer_slot_idx"]
        for t in range(Ts[s]):
            lanes = eo.rank_lanes(idxs[s][t], L, E)
            for k in range(K):
                d = next((r for r, kk in lanes.items() if kk == k), None)
                if d is None:
                    assert int(slot[t, k]) == -1
                    continue
                rows = [(int(v) // M, int(v) % M) for v in outs[d]["recv_src_metadata"][:, 0].tolist()]
                begin = next(i for i, (q, _) in enumerate(rows) if q == s)
                assert int(slot[t, k]) - s * M == rows.index((s, t)) - begin


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"R{c[0]}_E{c[3]}_K{c[4]}_a{c[7]}")
def test_combine_closed_forms(case):
    """Identity experts: the flat layout returns x times the number of ranks a
    token reached, the expanded layout x times the number of experts it chose
    (small integers: exact in bf16 arithmetic for integer-valued x)."""
    R, Ts, H, E, K, M, kind, align = case
    L = E // R
    ins = [make_rank_inputs(78, r, Ts[r], H, E, K, kind, n_mask=5) for r in range(R)]
    idxs = [i[1] for i in ins]
    g = torch.Generator().manual_seed(3)
    xs = [torch.randint(-8, 9, (Ts[r], H), generator=g).to(torch.bfloat16) for r in range(R)]
    for expand in (False, True):
        outs = eo.elastic_dispatch(xs, idxs, None, E, M, align, expand)
        comb = eo.elastic_combine([o["recv_x"] for o in outs], outs, idxs, E, expand)
        for s in range(R):
            valid = ((idxs[s] >= 0) & (idxs[s] < E))
            reached = torch.tensor([len(eo.rank_lanes(idxs[s][t], L, E)) for t in range(Ts[s])])
            factor = valid.sum(1) if expand else reached
            want = (xs[s].float() * factor.view(-1, 1).float()).to(torch.bfloat16)
            assert torch.equal(comb[s], want), (s, expand)
    # nothing in, nothing out; a token without valid choices combines to zeros
    zero = eo.elastic_combine([torch.zeros_like(o["recv_x"]) for o in outs], outs, idxs, E, True)
    assert all(float(z.abs().sum()) == 0.0 for z in zero)
