"""Size-independent properties of the CPU oracle on random small groups: what
goes in comes out exactly once, in the canonical order, and combine of the
untouched payload is the weighted sum. These are the same properties the GPU
tests use at full size, checked here on the checker itself."""
import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

from oracle import ep_oracle as ora


def _group(seed, R, L, K, H, tokens, n_mask):
    g = torch.Generator().manual_seed(seed)
    E = R * L
    xs, idxs, ws = [], [], []
    for r in range(R):
        T = tokens[r]
        x = torch.randn((T, H), generator=g).to(torch.bfloat16)
        idx = torch.topk(torch.randn((T, E), generator=g), K, dim=-1)[1].to(torch.int64).contiguous()
        w = torch.rand((T, K), generator=g).float().contiguous()
        for _ in range(n_mask if T else 0):
            idx[int(torch.randint(0, T, (1,), generator=g)), int(torch.randint(0, K, (1,), generator=g))] = -1
        xs.append(x), idxs.append(idx), ws.append(w)
    return xs, idxs, ws, E


cfg = st.tuples(st.integers(0, 10_000), st.integers(1, 4), st.integers(1, 5), st.integers(1, 4),
                st.sampled_from([128, 256, 640]), st.integers(0, 6))


@settings(max_examples=40, deadline=None)
@given(cfg, st.data())
def test_dispatch_is_a_permutation_in_canonical_order(c, data):
    seed, R, L, K, H, n_mask = c
    K = min(K, R * L)
    M = 12
    tokens = [data.draw(st.integers(0, M)) for _ in range(R)]
    xs, idxs, ws, E = _group(seed, R, L, K, H, tokens, n_mask)
    res = ora.dispatch(xs, idxs, M, E, False)
    seen = 0
    for r in range(R):
        out = res[r]
        assert int(out["recv_count"].sum()) == int(sum((idxs[s] // L == r).sum() for s in range(R)))
        for le in range(L):
            e = r * L + le
            n = int(out["recv_count"][le])
            lr = out["layout_range"][le]
            assert int((lr & 0xFFFFFFFF).sum()) == n
            row = 0
            for s in range(R):
                begin, cnt = int(lr[s] >> 32), int(lr[s] & 0xFFFFFFFF)
                want = [t for t in range(tokens[s]) if (idxs[s][t] == e).any()]
                assert cnt == len(want)
                if cnt:
                    assert begin == row
                    got = out["src_info"][le, begin:begin + cnt].tolist()
                    assert got == want  # token-ascending inside a source
                    for j, t in enumerate(want):
                        assert torch.equal(out["recv_x"][le, begin + j].view(torch.int16),
                                           xs[s][t].view(torch.int16))
                else:
                    assert int(lr[s]) == 0
                row += cnt
            seen += n
    assert seen == int(sum((i >= 0).sum() for i in idxs))


@settings(max_examples=25, deadline=None)
@given(cfg, st.data())
def test_combine_of_the_untouched_payload_is_the_weighted_sum(c, data):
    seed, R, L, K, H, n_mask = c
    K = min(K, R * L)
    M = 10
    tokens = [data.draw(st.integers(0, M)) for _ in range(R)]
    xs, idxs, ws, E = _group(seed, R, L, K, H, tokens, n_mask)
    res = ora.dispatch(xs, idxs, M, E, False)
    ys = [r_["recv_x"] for r_ in res]
    out32 = ora.combine(ys, idxs, ws, res, M, E, want_f32=True)
    out16 = ora.combine(ys, idxs, ws, res, M, E)
    for r in range(R):
        wsum = ws[r].masked_fill(idxs[r] < 0, 0).sum(dim=1, keepdim=True)
        want = xs[r].float() * wsum
        if want.numel() == 0:
            assert out16[r].numel() == 0
            continue
        scale = float(want.abs().max().clamp_min(1e-6))
        assert float((out32[r] - want).abs().max()) <= 2e-6 * scale * K + 1e-12
        assert float((out16[r].float() - want).abs().max()) <= 1e-2 * scale


@settings(max_examples=25, deadline=None)
@given(st.integers(0, 10_000), st.integers(1, 9), st.sampled_from([128, 384, 1024]))
def test_fp8_quantisation_properties(seed, n, H):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((n, H), generator=g) * float(torch.rand((), generator=g) * 50 + 1e-3)).to(torch.bfloat16)
    q, s = ora.fp8_quant(x)
    assert q.dtype == torch.uint8 and q.shape == (n, H) and s.shape == (n, H // 128)
    amax = x.float().abs().view(n, H // 128, 128).amax(dim=-1).clamp_min(1e-4)
    assert torch.equal(s, amax * np.float32(1.0 / 448.0))           # the kernel's formula, bit for bit
    assert int((q & 0x7F).max()) <= 0x7E                           # finite codes only (saturating)
    back = ora.fp8_dequant(q, s).float()
    # e4m3 keeps 3 mantissa bits: half an ulp is 2^-4 relative, plus the bf16 rounding of the result
    err = (back - x.float()).abs().view(n, H // 128, 128)
    assert bool((err <= amax.unsqueeze(-1) * (2.0 ** -4) + 1e-6).all())
    # quantising the same rows again gives the same bytes
    q2, s2 = ora.fp8_quant(x.clone())
    assert torch.equal(q, q2) and torch.equal(s, s2)
