"""Property tests of the numpy oracle (CPU): routing invariants over random shapes and
scores, including heavy ties, and algebraic properties of the linear stages."""
import numpy as np
from hypothesis import given, settings, strategies as st

from oracle import moe_oracle as orc


@settings(max_examples=60, deadline=None)
@given(T=st.integers(1, 70), E=st.integers(1, 40), kk=st.integers(1, 40), seed=st.integers(0, 10 ** 6),
       levels=st.integers(1, 6))
def test_routing_invariants_with_ties(T, E, kk, seed, levels):
    k = min(kk, E)
    rng = np.random.default_rng(seed)
    # few distinct score values -> many ties; the rule must stay deterministic and stable
    sc = rng.integers(0, levels, size=(T, E)).astype(np.float32)
    x = rng.standard_normal((T, 3)).astype(np.float32)
    xe, ew, inv, off = orc.moe_select(x, sc, E, k)
    vals, idx = orc.topk_desc(sc, k)
    assert np.all(np.diff(vals, axis=1) <= 0)                                   # descending
    for t in range(T):
        assert len(set(idx[t].tolist())) == k                                    # distinct experts
        rest = np.delete(sc[t], idx[t])
        assert rest.size == 0 or rest.max() <= vals[t].min()                     # really the top k
        for a in range(k - 1):                                                   # equal scores: lower index first
            if vals[t, a] == vals[t, a + 1]:
                assert idx[t, a] < idx[t, a + 1]
    assert off[0] == 0 and off[-1] == T * k and np.all(np.diff(off) >= 0)
    assert sorted(inv.reshape(-1).tolist()) == list(range(T * k))
    assert np.array_equal(xe[inv.reshape(-1)], np.repeat(x, k, axis=0))
    counts = np.bincount(idx.reshape(-1), minlength=E)
    assert np.array_equal(np.diff(off), counts)
    slot_of_row = np.argsort(inv.reshape(-1))
    for e in range(E):
        seg = slot_of_row[off[e]:off[e + 1]]
        assert np.all(np.diff(seg) > 0)                                          # stable inside an expert
        assert np.all(idx.reshape(-1)[seg] == e)
    np.testing.assert_allclose(ew.sum(1), 1.0, atol=1e-5)


@settings(max_examples=25, deadline=None)
@given(seed=st.integers(0, 10 ** 6), E=st.integers(1, 6), K=st.integers(1, 20), N=st.integers(1, 12))
def test_grouped_linear_is_linear_and_blockwise(seed, E, K, N):
    rng = np.random.default_rng(seed)
    M = int(rng.integers(1, 40))
    cuts = np.sort(rng.integers(0, M + 1, E - 1)) if E > 1 else np.array([], int)
    off = np.concatenate([[0], cuts, [M]]).astype(np.int64)
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = rng.standard_normal((E, N, K)).astype(np.float32)
    y = orc.moe_grouped_linear(x, off, w)
    np.testing.assert_allclose(orc.moe_grouped_linear(2 * x, off, w), 2 * y, rtol=1e-6)
    for e in range(E):
        np.testing.assert_allclose(y[off[e]:off[e + 1]], x[off[e]:off[e + 1]] @ w[e].T, rtol=1e-4, atol=1e-5)
    # the combine undoes the dispatch when the weights of a token sum to one
    k = 2
    T = 7
    sc = rng.standard_normal((T, 5)).astype(np.float32)
    xt = rng.standard_normal((T, 4)).astype(np.float32)
    xe, ew, inv, _ = orc.moe_select(xt, sc, 5, k)
    np.testing.assert_allclose(orc.moe_reduce(xe, ew, inv, k), xt, rtol=1e-5, atol=1e-6)
