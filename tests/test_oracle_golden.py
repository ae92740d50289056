"""The numpy oracle against the golden vectors produced by the OPMX reference
operators (tests/golden/make_golden.py).  CPU only."""
import glob
import json
import os

import numpy as np
import pytest

from oracle import moe_oracle as orc

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
ATOL, RTOL = 2e-2, 1e-2          # parity tolerance for fp16/bf16 results


def load(name):
    return dict(np.load(os.path.join(GOLDEN, name), allow_pickle=False))


def ulp_close(a, b, dtype, ulps=None):
    """|a-b| <= `ulps` units in the last place of `dtype`.  Default: 1 ulp for
    fp16/bf16 (one rounding of an fp32 softmax), 4 ulp for fp32 (different exp
    implementations)."""
    if ulps is None:
        ulps = 4 if dtype == "f32" else 1
    eps = {"f32": 2.0 ** -23, "f16": 2.0 ** -10, "bf16": 2.0 ** -7}[dtype]
    return np.all(np.abs(a - b) <= ulps * eps * np.maximum(np.abs(a), np.abs(b)) + 1e-30)


SELECT = sorted(os.path.basename(p) for p in glob.glob(os.path.join(GOLDEN, "select_*.npz")))


@pytest.mark.parametrize("name", SELECT)
def test_select_matches_reference(name):
    g = load(name)
    dtype, E, k = str(g["dtype"]), int(g["E"]), int(g["k"])
    H = g["x"].shape[-1]
    x = g["x"].reshape(-1, H)
    sc = g["scores"].reshape(-1, E)
    assert not orc.rows_with_ties(sc, k).any()
    xe, ew, inv, off = orc.moe_select(x, sc, E, k, dtype)
    assert np.array_equal(off, g["expert_offset"])
    assert np.array_equal(inv.reshape(-1), g["invert_permutation"].reshape(-1))
    assert np.array_equal(xe, g["x_expand_permute"].reshape(-1, H))
    assert ulp_close(ew.reshape(-1), g["expert_weights"].reshape(-1), dtype)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_linears_and_activations_match_reference(dtype):
    g = load(f"linear_{dtype}.npz")
    x = g["x"].reshape(-1, g["x"].shape[-1])
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == "f32" else dict(atol=ATOL, rtol=RTOL)
    for tag in ("arange", "ragged"):
        off = g["off_" + tag]
        y = orc.moe_grouped_linear(x, off, g["w"], g["b"])
        np.testing.assert_allclose(y, g["col_bias_" + tag].reshape(y.shape), **tol)
        y = orc.moe_grouped_linear(x, off, g["w"])
        np.testing.assert_allclose(y, g["col_nobias_" + tag].reshape(y.shape), **tol)
        np.testing.assert_allclose(y, g["row_nobias_" + tag].reshape(y.shape), **tol)
        # rows outside [off[0], off[E]) are zero in the reference and the oracle
        ref = g["col_bias_" + tag].reshape(y.shape)
        outside = np.ones(y.shape[0], bool)
        outside[off[0]:off[-1]] = False
        assert not ref[outside].any() and not y[outside].any()
    np.testing.assert_allclose(orc.swiglu(g["swiglu_in"]), g["swiglu_out"], **tol)
    np.testing.assert_allclose(orc.swiglu(g["swiglu_in"], 1.7), g["swiglu_out_beta"], **tol)
    d = g["swiglu_in"].shape[-1] // 2
    a, c = g["swiglu_in"][..., :d], g["swiglu_in"][..., d:]
    np.testing.assert_allclose(orc.silu_gate(a, c), g["silu_gate_out"], **tol)
    np.testing.assert_allclose(orc.silu_gate(a), g["silu_out"], **tol)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_reduce_matches_reference(dtype):
    g = load(f"reduce_{dtype}.npz")
    k = int(g["k"])
    N = g["y"].shape[-1]
    out = orc.moe_reduce(g["y"].reshape(-1, N), g["expert_weights"], g["invert_permutation"], k)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == "f32" else dict(atol=ATOL, rtol=RTOL)
    np.testing.assert_allclose(out, g["out"], **tol)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_rms_norm_matches_reference(dtype):
    g = load(f"rmsnorm_{dtype}.npz")
    ulp = {"f32": 2.0 ** -22, "f16": 2.0 ** -9, "bf16": 2.0 ** -6}[dtype]      # 2 ulp: rsqrt and two roundings
    y, s = orc.skip_rms_norm(g["x"], g["weight"], g["skip"], 1e-5, dtype)
    assert np.array_equal(s, g["skip_out"])
    np.testing.assert_allclose(y, g["y_skip"], rtol=ulp, atol=1e-6)
    y, s = orc.skip_rms_norm(g["x"], g["weight"], None, 1e-6, dtype)
    assert np.array_equal(s, g["x"])
    np.testing.assert_allclose(y, g["y_noskip"], rtol=ulp, atol=1e-6)
    np.testing.assert_allclose(orc.skip_rms_norm(g["x"], g["weight"], None, 1e-5, dtype)[0], g["y_plain"], rtol=ulp, atol=1e-6)


@pytest.mark.parametrize("name", ["block_f32", "block_f16", "block_bf16", "block_f16_fine"])
def test_block_matches_reference(name):
    g = load(name + ".npz")
    dtype, E, k = str(g["dtype"]), int(g["E"]), int(g["k"])
    # routing is compared on the reference's own scores (its gate linear rounds
    # through the CPU BLAS, which the oracle does not model bit for bit)
    r = orc.moe_block(g["x"], g["w_router"], g["w_gate_up"], g["w_down"], E, k, dtype,
                      scores=g["scores"])
    tied = orc.rows_with_ties(g["scores"], k)
    assert int(tied.sum()) == int(g["tied_rows"])
    if not tied.any():
        assert np.array_equal(r["expert_offset"], g["expert_offset"])
        assert np.array_equal(r["invert_permutation"], g["invert_permutation"])
        assert np.array_equal(r["x_expand_permute"], g["x_expand_permute"].reshape(r["x_expand_permute"].shape))
        assert ulp_close(r["expert_weights"], g["expert_weights"], dtype)
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == "f32" else dict(atol=ATOL, rtol=RTOL)
    if not tied.any():
        for key in ("x13", "h", "y"):
            np.testing.assert_allclose(r[key], g[key].reshape(r[key].shape), err_msg=key, **tol)
    np.testing.assert_allclose(r["out"], g["out"], **tol)
    np.testing.assert_allclose(r["out"], g["out_fp32_reference"], **tol)
    # the gate linear restated in the oracle agrees with the reference's scores
    s = orc.moe_block(g["x"], g["w_router"], g["w_gate_up"], g["w_down"], E, k, dtype)["scores"]
    np.testing.assert_allclose(s, g["scores"], atol=2e-3, rtol=1e-2)


def test_tie_rule_is_deterministic_and_lowest_index_first():
    s = np.array([[1, 1, 1, 1, .5, 1, 1, 1], [0.0, -0.0, -1, -1, -2, -3, -4, -5]], np.float32)
    v, i = orc.topk_desc(s, 2)
    assert i.tolist() == [[0, 1], [0, 1]]
    assert orc.rows_with_ties(s, 2).tolist() == [True, True]
    d, n = orc.detie_scores(s, "f16")
    assert n > 0 and not orc.rows_with_ties(d, 7).any()


def test_select_invariants_random():
    rng = np.random.default_rng(0)
    for T, E, k in [(1, 8, 2), (257, 8, 2), (100, 64, 8), (31, 5, 5)]:
        x = rng.standard_normal((T, 8)).astype(np.float32)
        sc = rng.standard_normal((T, E)).astype(np.float32)
        xe, ew, inv, off = orc.moe_select(x, sc, E, k)
        assert off[0] == 0 and off[-1] == T * k and np.all(np.diff(off) >= 0)
        assert sorted(inv.reshape(-1).tolist()) == list(range(T * k))
        assert np.array_equal(xe[inv.reshape(-1)], np.repeat(x, k, axis=0))
        np.testing.assert_allclose(ew.sum(1), 1.0, atol=1e-6)
        # stability: inside an expert rows keep ascending flat-slot order
        slot_of_row = np.argsort(inv.reshape(-1))
        for e in range(E):
            seg = slot_of_row[off[e]:off[e + 1]]
            assert np.all(np.diff(seg) > 0)


def test_onnx_fixture_lists_the_five_nodes():
    with open(os.path.join(GOLDEN, "onnx_block_graph.json")) as f:
        nodes = json.load(f)["nodes"]
    assert [n["kind"] for n in nodes] == [
        "opmx::MoeSelect", "opmx::MoeColumnParallelLinear", "opmx::SwiGLU",
        "opmx::MoeRowParallelLinear", "opmx::MoeReduce"]


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_dense_linear_matches_reference(dtype):
    g = load(f"dense_linear_{dtype}.npz")
    tol = dict(atol=2e-5, rtol=1e-5) if dtype == "f32" else dict(atol=2e-2, rtol=1e-2)
    y = orc.linear(g["x"], g["w"])
    np.testing.assert_allclose(y, g["linear"], **tol)
    yb = orc.linear(g["x"], g["w"], g["b"])
    for name in ("linear_bias", "column", "row"):
        np.testing.assert_allclose(yb, g[name], err_msg=name, **tol)
    np.testing.assert_allclose(yb, g["linear_bias_fp32"], atol=2e-5, rtol=1e-5)


def attention_fixture(name):
    """-> (fixture dict, cache_in, cache_out) with the caches as float32 values."""
    g = load(name)
    conv = (lambda a: a.astype(np.float32)) if str(g["dtype"]) == "f16" else orc.bf16_bits_to_f32
    return g, conv(g["cache_in"]), conv(g["cache_out"])


ATTN = [f"attn_decode_f16_layout{l}.npz" for l in range(4)] + [f"attn_decode_bf16_layout{l}.npz" for l in (0, 3)]


@pytest.mark.parametrize("name", ATTN)
def test_decode_cache_attention_matches_reference(name):
    g, cache, cache_out = attention_fixture(name)
    out = orc.decode_cache_attention(g["q"], g["k"], g["v"], cache, g["cachestarts"], g["start_pos"],
                                     int(g["layout"]), int(g["layer_idx"]))
    assert np.array_equal(cache, cache_out), "the new keys / values must land where the reference puts them"
    # the reference rounds the probabilities to the cache dtype before the value product
    np.testing.assert_allclose(out, g["out"], atol=2e-2, rtol=1e-2)
