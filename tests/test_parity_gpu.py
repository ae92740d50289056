"""Parity of the CUDA path, called through the C ABI, with the CPU oracle and
with the golden vectors the OPMX reference operators produced.

Integer results (expert_offset, invert_permutation, the gathered rows) must be
bit-exact; expert_weights within 1 ulp of one rounding of the fp32 softmax;
fp16/bf16 GEMM results within max-abs 2e-2 / rel 1e-2 of the fp32 reference.
"""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from tests.helpers import GOLDEN, TAG, assert_close, assert_ulp, dev, host, load

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def F():
    import ppl.pmx_b200.torch_function as F
    return F


def gpu_select(F, x, sc, E, k, dtype):
    xe, ew, inv, off = F.moe_select(dev(x, dtype), dev(sc, dtype), E, k)
    torch.cuda.synchronize()
    return xe, ew, inv, off


def check_select(F, x, sc, E, k, dtype, golden=None):
    H = x.shape[-1]
    xe, ew, inv, off = gpu_select(F, x, sc, E, k, dtype)
    assert inv.dtype == torch.int64 and off.dtype == torch.int64
    assert tuple(xe.shape) == (*x.shape[:-1], k, H) and tuple(ew.shape) == (*x.shape[:-1], k)
    oxe, oew, oinv, ooff = orc.moe_select(x.reshape(-1, H), sc.reshape(-1, E), E, k, dtype)
    assert np.array_equal(off.cpu().numpy(), ooff)
    assert np.array_equal(inv.cpu().numpy().reshape(-1), oinv.reshape(-1))
    assert np.array_equal(host(xe).reshape(-1, H), oxe)
    assert_ulp(ew.reshape(-1), oew.reshape(-1), dtype, msg="expert_weights vs oracle")
    if golden is not None:
        assert np.array_equal(off.cpu().numpy(), golden["expert_offset"])
        assert np.array_equal(inv.cpu().numpy(), golden["invert_permutation"])
        assert np.array_equal(host(xe), golden["x_expand_permute"])
        assert_ulp(ew, golden["expert_weights"], dtype, msg="expert_weights vs reference")
    return xe, ew, inv, off


SELECT = sorted(os.path.basename(p) for p in glob.glob(os.path.join(GOLDEN, "select_*.npz")))


@pytest.mark.parametrize("name", SELECT)
def test_select_golden(F, name):
    g = load(name)
    check_select(F, g["x"], g["scores"], int(g["E"]), int(g["k"]), str(g["dtype"]), golden=g)


@pytest.mark.parametrize("T,H,E,k,dtype", [
    (1, 8, 8, 2, "f16"), (2, 24, 8, 2, "bf16"), (17, 5, 3, 1, "f32"), (300, 40, 8, 2, "f16"),
    (513, 16, 64, 8, "f16"), (4097, 8, 8, 2, "bf16"), (64, 7, 8, 8, "f32"), (1000, 3, 160, 6, "f16"),
    (9000, 8, 32, 32, "bf16"),
    # the one-launch path for large batches (<= 64 experts), its limits, and the three-launch
    # path behind it (more than 64 experts, or more than 1024 tokens per SM)
    (5000, 64, 64, 8, "f16"), (20000, 16, 8, 2, "f32"), (1025, 24, 5, 5, "bf16"), (3000, 8, 70, 3, "f16"),
    (160000, 8, 8, 2, "f16"),
])
def test_select_random_shapes(F, T, H, E, k, dtype):
    rng = np.random.default_rng(T * 7 + E)
    x = orc.round_to_dtype(rng.standard_normal((T, H)).astype(np.float32), dtype)
    sc, _ = orc.detie_scores(rng.standard_normal((T, E)).astype(np.float32), dtype)
    check_select(F, x, sc, E, k, dtype)


def test_select_ties_follow_the_stated_rule(F):
    # equal scores: higher score first, lower expert index among equals (not torch.topk's
    # implementation-defined order); -0.0 ties with +0.0
    sc = np.array([[1, 1, 1, 1, .5, 1, 1, 1], [0.0, -0.0, -1, -1, -2, -3, -4, -5],
                   [3, 3, 3, 3, 3, 3, 3, 3], [-1, 2, 2, -1, 2, 0, 0, 7]], np.float32)
    x = np.arange(4 * 8, dtype=np.float32).reshape(4, 8)
    for dtype in ("f16", "bf16", "f32"):
        for k in (1, 2, 3, 8):
            check_select(F, x, sc, 8, k, dtype)


def test_select_all_tokens_to_one_expert_and_empty_experts(F):
    T, E = 257, 16
    sc = np.full((T, E), -1e4, np.float32)
    sc[:, 5] = 3.0
    sc[:, 11] = 1.0
    x = np.random.default_rng(1).standard_normal((T, 32)).astype(np.float16).astype(np.float32)
    sc2, _ = orc.detie_scores(sc, "f16")
    xe, ew, inv, off = check_select(F, x, sc2, E, 2, "f16")
    counts = np.diff(off.cpu().numpy())
    assert counts[5] == T and counts[11] == T and counts.sum() == 2 * T


def test_select_leading_dims_and_noncontiguous_input(F):
    rng = np.random.default_rng(3)
    x = orc.round_to_dtype(rng.standard_normal((3, 5, 64)).astype(np.float32), "f16")
    sc, _ = orc.detie_scores(rng.standard_normal((15, 8)).astype(np.float32), "f16")
    sc = sc.reshape(3, 5, 8)
    check_select(F, x, sc, 8, 2, "f16")
    xt = dev(x.reshape(15, 64), "f16").t().contiguous().t()      # non-contiguous view
    assert not xt.is_contiguous()
    xe, ew, inv, off = F.moe_select(xt, dev(sc.reshape(15, 8), "f16"), 8, 2)
    oxe, _, oinv, ooff = orc.moe_select(x.reshape(15, 64), sc.reshape(15, 8), 8, 2, "f16")
    assert np.array_equal(host(xe).reshape(-1, 64), oxe) and np.array_equal(inv.cpu().numpy(), oinv)


@pytest.mark.parametrize("T,H,E,k,dtype", [(1, 4096, 8, 2, "f16"), (64, 4096, 8, 2, "f16"), (300, 512, 8, 2, "bf16"),
                                            (1024, 256, 64, 8, "f16"), (77, 64, 5, 3, "f32"), (500, 128, 16, 16, "bf16")])
def test_route_select_fused_router(F, T, H, E, k, dtype):
    """Router gate + select in one launch: the scores it returns match the gate linear, and
    the routing is bit-exact for exactly those scores."""
    rng = np.random.default_rng(T + E)
    x = orc.round_to_dtype(rng.standard_normal((T, H)).astype(np.float32), dtype)
    wr = orc.round_to_dtype((rng.standard_normal((E, H)) * 0.02).astype(np.float32), dtype)
    for rep in range(2):
        out = F.moe_route_select(dev(x, dtype), dev(wr, dtype), E, k)
        assert out is not None
        sc, xe, ew, inv, off = out
        torch.cuda.synchronize()
        ref_scores = (x.astype(np.float64) @ wr.astype(np.float64).T).astype(np.float32)
        assert_close(sc, ref_scores, dtype, "router scores")
        s32 = host(sc)
        oxe, oew, oinv, ooff = orc.moe_select(x, s32, E, k, dtype)
        tied = orc.rows_with_ties(s32, k)
        if not tied.any():
            assert np.array_equal(off.cpu().numpy(), ooff)
            assert np.array_equal(inv.cpu().numpy(), oinv)
            assert np.array_equal(host(xe).reshape(-1, H), oxe)
            assert_ulp(ew, oew, dtype, msg="expert_weights")
        # the stand-alone moe_select on the same scores gives the same result in any case
        xe2, ew2, inv2, off2 = F.moe_select(dev(x, dtype), sc, E, k)
        assert torch.equal(off, off2) and torch.equal(inv, inv2) and torch.equal(xe, xe2) and torch.equal(ew, ew2)
    assert F.moe_route_select(torch.zeros(2000, 64, device="cuda", dtype=torch.float16),
                              torch.zeros(8, 64, device="cuda", dtype=torch.float16), 8, 2) is None


@pytest.mark.parametrize("T,H,E,k,dtype,with_skip", [(1, 4096, 8, 2, "f16", True), (64, 4096, 8, 2, "f16", True),
                                                      (64, 4096, 8, 2, "bf16", False), (700, 512, 64, 8, "f16", True),
                                                      (33, 64, 5, 3, "f32", True)])
def test_norm_route_select_fused_front_end(F, T, H, E, k, dtype, with_skip):
    """skip_rms_norm + router gate + select in one launch: the residual stream is bit-exact,
    the normalised rows it routes are within 3 ulp of the oracle, the scores match the gate
    linear of those rows and the routing is bit-exact for exactly those scores."""
    rng = np.random.default_rng(T + E + H)
    x = orc.round_to_dtype(rng.standard_normal((T, H)).astype(np.float32) * 2, dtype)
    sk = orc.round_to_dtype(rng.standard_normal((T, H)).astype(np.float32), dtype) if with_skip else None
    nw = orc.round_to_dtype(1 + 0.1 * rng.standard_normal(H).astype(np.float32), dtype)
    wr = orc.round_to_dtype((rng.standard_normal((E, H)) * 0.05).astype(np.float32), dtype)
    out = F.moe_norm_route_select(dev(x, dtype), dev(sk, dtype) if with_skip else None, dev(nw, dtype), 1e-5,
                                  dev(wr, dtype), E, k)
    assert out is not None
    h, sc, xe, ew, inv, off = out
    torch.cuda.synchronize()
    oy, os_ = orc.skip_rms_norm(x, nw, sk, 1e-5, dtype)
    assert np.array_equal(host(h), os_)
    ulp = 1.5 * {"f32": 2.0 ** -22, "f16": 2.0 ** -9, "bf16": 2.0 ** -6}[dtype]
    rows = host(xe).reshape(-1, H)[inv.cpu().numpy().reshape(-1)].reshape(T, k, H)   # slot (t, j) -> its row
    for j in range(k):
        np.testing.assert_allclose(rows[:, j], oy, rtol=ulp, atol=1e-6)
    n_gpu = rows[:, 0]                                       # the normalised rows the kernel used
    ref_scores = (n_gpu.astype(np.float64) @ wr.astype(np.float64).T).astype(np.float32)
    assert_close(sc, ref_scores, dtype, "router scores")
    s32 = host(sc)
    if not orc.rows_with_ties(s32, k).any():
        oxe, oew, oinv, ooff = orc.moe_select(n_gpu, s32, E, k, dtype)
        assert np.array_equal(off.cpu().numpy(), ooff) and np.array_equal(inv.cpu().numpy(), oinv)
        assert np.array_equal(host(xe).reshape(-1, H), oxe)
        assert_ulp(ew, oew, dtype, msg="expert_weights")
    assert F.moe_norm_route_select(torch.zeros(2000, 64, device="cuda", dtype=torch.float16), None,
                                   torch.ones(64, device="cuda", dtype=torch.float16), 1e-5,
                                   torch.zeros(8, 64, device="cuda", dtype=torch.float16), 8, 2) is None


def test_block_from_residual(F):
    """MoeFeedForward.forward_from_residual (norm + block; fused front end for a decode batch,
    stand-alone operators for a large one) against the oracle chain."""
    from ppl.pmx_b200 import workloads as W
    from ppl.pmx_b200.moe_layers import MoeFeedForward
    for wl, kw in (("decode_t64", dict(H=512, I=1024)), ("prefill", dict(T=1500, H=256, I=512))):
        sh = W.scaled(W.WORKLOADS[wl], **kw)
        x, wr, _, _ = W.make_activations(sh)
        g = torch.Generator().manual_seed(3)
        skip = torch.randn(sh.T, sh.H, generator=g).to(x.dtype)
        nw = (1 + 0.1 * torch.randn(sh.H, generator=g)).to(x.dtype)
        wu, w2 = W.make_expert_weights(sh, "cuda")
        blk = MoeFeedForward(sh.H, sh.I, sh.E, sh.k, None, False).cuda().to(W.TORCH_DTYPE[sh.dtype])
        with torch.no_grad():
            blk.gate.weight.copy_(wr)
            blk.wu.weight.copy_(wu)
            blk.w2.weight.copy_(w2)
            out, h = blk.forward_from_residual(x.cuda(), skip.cuda(), nw.cuda(), 1e-5)
            norm, h2 = F.skip_rms_norm(x.cuda(), nw.cuda(), skip.cuda(), -1, 1e-5)
            fused = F.moe_norm_route_select(x.cuda(), skip.cuda(), nw.cuda(), 1e-5, blk.gate.weight, sh.E, sh.k)
            sc = fused[1] if fused is not None else torch.nn.functional.linear(norm, blk.gate.weight)
        assert torch.equal(h, h2)
        oy, _ = orc.skip_rms_norm(host(x), host(nw), host(skip), 1e-5, sh.dtype)
        r = orc.moe_block(oy, host(wr), host(wu), host(w2), sh.E, sh.k, sh.dtype, scores=host(sc),
                          round_intermediates=False)
        assert_close(out, r["out"], sh.dtype, wl)


def test_select_errors(F):
    x = torch.randn(4, 8, device="cuda", dtype=torch.float16)
    s = torch.randn(4, 8, device="cuda", dtype=torch.float16)
    with pytest.raises(ValueError):
        F.moe_select(x, s, 8, 9)                      # k > E
    with pytest.raises(ValueError):
        F.moe_select(x[:0], s[:0], 8, 2)              # no tokens
    with pytest.raises(ValueError):
        F.moe_select(x, s[:, :4], 8, 2)               # scores width
    with pytest.raises(RuntimeError):
        F.moe_select(x.cpu(), s.cpu(), 8, 2)          # no CPU fallback
    with pytest.raises(TypeError):
        F.moe_select(x.double(), s.double(), 8, 2)


# --------------------------------------------------------------------------- linears
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_linear_golden(F, dtype):
    g = load(f"linear_{dtype}.npz")
    E, N, K = g["w"].shape
    x, w, b = dev(g["x"], dtype), dev(g["w"], dtype), dev(g["b"], dtype)
    for tag in ("arange", "ragged"):
        off = torch.from_numpy(g["off_" + tag])
        y = F.moe_column_parallel_linear(x, off, w, b, None, E, K, N, False)
        assert y.dtype == x.dtype and y.shape == (*x.shape[:-1], N)
        assert_close(y, g["col_bias_" + tag], dtype, "col bias " + tag)
        y = F.moe_column_parallel_linear(x, off.to(torch.int32).cuda(), w, None, None, E, K, N, True)
        assert_close(y, g["col_nobias_" + tag], dtype, "col " + tag)
        y = F.moe_row_parallel_linear(x, off.cuda(), w, None, None, E, K, N, True)
        assert_close(y, g["row_nobias_" + tag], dtype, "row " + tag)
        # rows no expert owns are exactly zero
        outside = np.ones(x.shape[0] * x.shape[1], bool)
        outside[g["off_" + tag][0]:g["off_" + tag][-1]] = False
        assert not host(y).reshape(-1, N)[outside].any()
    assert_close(F.swiglu(dev(g["swiglu_in"], dtype)), g["swiglu_out"], dtype)
    assert_close(F.swiglu(dev(g["swiglu_in"], dtype), 1.7), g["swiglu_out_beta"], dtype)
    d = g["swiglu_in"].shape[-1] // 2
    a, c = dev(g["swiglu_in"][..., :d], dtype), dev(g["swiglu_in"][..., d:], dtype)
    assert_close(F.silu(a, c), g["silu_gate_out"], dtype)
    assert_close(F.silu(a), g["silu_out"], dtype)


def ragged_offsets(rng, M, E, empty=2, lead=0, trail=0):
    cuts = np.sort(rng.integers(lead, M - trail + 1, E - 1))
    off = np.concatenate([[lead], cuts, [M - trail]]).astype(np.int64)
    for e in rng.choice(E, size=min(empty, E - 1), replace=False):
        off[e + 1] = off[e]
    return np.maximum.accumulate(off)


def run_linear(F, rng, M, N, K, E, dtype, plan=None, bias=False, swiglu=False, off=None):
    from ppl.pmx_b200._cabi import GemmPlan
    from ppl.pmx_b200.torch_function.moe import moe_grouped_linear, grouped_linear_check
    x = orc.round_to_dtype(rng.standard_normal((M, K)).astype(np.float32), dtype)
    w = orc.round_to_dtype((rng.standard_normal((E, N, K)) / np.sqrt(K)).astype(np.float32), dtype)
    b = orc.round_to_dtype(rng.standard_normal((E, N)).astype(np.float32), dtype) if bias else None
    if off is None:
        off = ragged_offsets(rng, M, E)
    p = GemmPlan(**plan) if plan else None
    y, ws = moe_grouped_linear(dev(x, dtype), torch.from_numpy(off).cuda(), dev(w, dtype),
                               dev(b, dtype) if bias else None, swiglu=swiglu, plan=p,
                               return_workspace=True)
    grouped_linear_check(ws)
    ref = orc.moe_grouped_linear(x, off, w, b)
    if swiglu:
        ref = orc.swiglu(ref)
    assert_close(y, ref, dtype, f"M={M} N={N} K={K} E={E} plan={plan}")
    return y


TC_SHAPES = [
    # M, N, K, E
    (64, 128, 64, 4), (200, 256, 128, 8), (300, 384, 192, 8), (1000, 512, 320, 8),
    (77, 136, 72, 3), (16, 1024, 512, 8), (2048, 256, 256, 2),
]


@pytest.mark.parametrize("M,N,K,E", TC_SHAPES)
@pytest.mark.parametrize("kernel", [1, 2, 3, 4])
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_grouped_linear_kernels(F, M, N, K, E, kernel, dtype):
    rng = np.random.default_rng(M + N + K + kernel)
    run_linear(F, rng, M, N, K, E, dtype, plan=dict(kernel=kernel), bias=(M % 2 == 0))


@pytest.mark.parametrize("M,N,K,E", TC_SHAPES)
@pytest.mark.parametrize("kernel", [1, 2, 3, 4])
def test_grouped_linear_swiglu_fused(F, M, N, K, E, kernel):
    from ppl.pmx_b200._cabi import PmxError
    rng = np.random.default_rng(M * 3 + N + K + kernel)
    args = (F, rng, M, N, K, E, "bf16" if kernel == 1 else "f16")
    kw = dict(plan=dict(kernel=kernel), bias=(M % 2 == 1), swiglu=True)
    if kernel != 3 and (N // 2) % 8:
        # the tensor-core kernels need 16-byte output rows; asking for one explicitly on
        # another shape is an error (the automatic choice uses the CUDA-core kernel)
        with pytest.raises(PmxError):
            run_linear(*args, **kw)
        run_linear(*args, bias=True, swiglu=True)
        return
    run_linear(*args, **kw)


@pytest.mark.parametrize("kernel,split", [(1, 2), (1, 3), (2, 4), (2, 7)])
def test_grouped_linear_split_k(F, kernel, split):
    rng = np.random.default_rng(split)
    off = ragged_offsets(rng, 90, 8, lead=5, trail=9)      # rows outside every expert -> zeros
    y = run_linear(F, rng, 90, 256, 1024, 8, "f16", plan=dict(kernel=kernel, split_k=split), bias=True, off=off)
    assert not host(y)[:5].any() and not host(y)[81:].any()


@pytest.mark.parametrize("kernel,split,M", [(2, 2, 16), (2, 4, 90), (1, 2, 300), (0, 0, 2), (0, 0, 40)])
def test_grouped_linear_split_k_with_swiglu_in_the_final_sum(F, kernel, split, M):
    """Few rows per expert: K is sliced, the kernel leaves fp32 [gate | up] partial sums and
    the activation is applied when they are added up.  (0, 0) = the automatic plan."""
    rng = np.random.default_rng(split + M)
    plan = dict(kernel=kernel, split_k=split) if kernel else None
    run_linear(F, rng, M, 512, 1024, 8, "f16", plan=plan, bias=True, swiglu=True,
               off=ragged_offsets(rng, M, 8, empty=3))
    run_linear(F, rng, M, 1024, 2048, 8, "bf16", plan=plan, swiglu=True)


@pytest.mark.parametrize("tile", [dict(kernel=4, tile_feat=32), dict(kernel=4, tile_feat=64, stages=2), dict(kernel=4, max_ctas=6),
                                  dict(kernel=4, tile_feat=256), dict(kernel=1, tile_feat=32), dict(kernel=1, tile_feat=64),
                                  dict(kernel=1, tile_feat=128, stages=2), dict(kernel=2, tile_tok=16),
                                  dict(kernel=2, tile_tok=64, stages=3), dict(kernel=2, tile_tok=256),
                                  dict(kernel=1, max_ctas=3), dict(kernel=2, max_ctas=1)])
def test_grouped_linear_tilings(F, tile):
    rng = np.random.default_rng(11)
    run_linear(F, rng, 333, 320, 256, 5, "bf16", plan=tile, bias=True)


@pytest.mark.parametrize("plan", [dict(kernel=2, stream_k=1), dict(kernel=2, stream_k=2), dict(kernel=1, stream_k=1),
                                  dict(kernel=2, stream_k=1, max_ctas=7), dict(kernel=2, stream_k=1, max_ctas=97),
                                  dict(kernel=1, stream_k=1, max_ctas=5, tile_feat=64),
                                  dict(kernel=2, stream_k=1, tile_tok=16, stages=8)])
@pytest.mark.parametrize("swiglu", [False, True])
def test_grouped_linear_stream_k(F, plan, swiglu):
    """k-blocks dealt out evenly over the CTAs: tiles cut at arbitrary k are finished by
    their owner from the partial tiles the following CTAs leave in the workspace."""
    rng = np.random.default_rng(len(str(plan)))
    for M, N, K, E in ((40, 512, 1024, 8), (3, 256, 4096, 8), (300, 384, 192, 4), (64, 1024, 64, 8)):
        run_linear(F, rng, M, N, K, E, "f16", plan=plan, bias=True, swiglu=swiglu)
    run_linear(F, rng, 130, 256, 2048, 6, "bf16", plan=plan, swiglu=swiglu)


def test_grouped_linear_stream_k_needs_one_cta_per_sm(F):
    """A stream-K plan whose shared-memory ring is so small that two CTAs would share an
    SM is refused (its CTAs wait for one another and must all be resident)."""
    from ppl.pmx_b200._cabi import PmxError
    with pytest.raises(PmxError):
        run_linear(F, np.random.default_rng(0), 40, 512, 1024, 8, "f16", plan=dict(kernel=2, stream_k=1, tile_tok=16, stages=2))


@pytest.mark.parametrize("plan", [dict(kernel=2), dict(kernel=2, balance=2), dict(kernel=2, cta_cap=5),
                                  dict(kernel=2, max_ctas=37), dict(kernel=2, tile_tok=16, cta_cap=148),
                                  dict(kernel=2, split_k=3), dict(kernel=2, balance=2, full_rounds=2, cta_cap=100)])
@pytest.mark.parametrize("swiglu", [False, True])
def test_grouped_linear_even_row_dealing(F, plan, swiglu):
    """Weight rows on MMA-M: the feature rows of all (expert, token tile) panels are dealt
    out in 8-row units, so items are ranges of 8..128 rows fetched as boxes of 64/32/16/8
    rows that may start anywhere; against whole 128-row tiles (balance=2)."""
    rng = np.random.default_rng(len(str(plan)) + swiglu)
    for M, N, K, E in ((40, 512, 1024, 8), (3, 3584, 512, 8), (300, 384, 192, 4), (64, 1040, 64, 8), (130, 2064, 320, 6)):
        run_linear(F, rng, M, N, K, E, "f16", plan=plan, bias=True, swiglu=swiglu)
    run_linear(F, rng, 70, 1808, 2048, 8, "bf16", plan=plan, swiglu=swiglu, off=ragged_offsets(rng, 70, 8, empty=3))


@pytest.mark.parametrize("M,dtype", [(40, "f16"), (700, "bf16"), (5000, "bf16"), (33, "f32")])
def test_grouped_linear_on_a_window_of_the_weight_rows(F, M, dtype):
    """W given as a strided window W_full[:, n0:n1, :] of a wider weight tensor (the hidden-column
    slices of the down projection): used in place through the expert row pitch, same result as
    the contiguous copy, on every kernel the automatic choice picks (decode, prefill, paired, fp32)."""
    from ppl.pmx_b200.torch_function.moe import moe_grouped_linear
    rng = np.random.default_rng(M)
    E, N_full, K = 4, 512, 256
    x = orc.round_to_dtype(rng.standard_normal((M, K)).astype(np.float32), dtype)
    w = orc.round_to_dtype((rng.standard_normal((E, N_full, K)) / np.sqrt(K)).astype(np.float32), dtype)
    b = orc.round_to_dtype(rng.standard_normal((E, N_full)).astype(np.float32), dtype)
    off = ragged_offsets(rng, M, E, empty=1)
    xd, wd, bd, od = dev(x, dtype), dev(w, dtype), dev(b, dtype), torch.from_numpy(off).cuda()
    for n0, n1 in ((0, 128), (128, 384), (384, 512)):
        ref = orc.moe_grouped_linear(x, off, w[:, n0:n1], b[:, n0:n1])
        window = wd[:, n0:n1, :]
        assert not window.is_contiguous() or n1 - n0 == N_full
        y = moe_grouped_linear(xd, od, window, bd[:, n0:n1])
        assert_close(y, ref, dtype, f"window [{n0},{n1})")
        assert torch.equal(y, moe_grouped_linear(xd, od, window.contiguous(), bd[:, n0:n1].contiguous()))


@pytest.mark.parametrize("T,H,E,k,N,dtype", [(64, 512, 8, 2, 1024, "f16"), (16, 256, 8, 2, 3584, "f16"),
                                             (100, 320, 16, 4, 528, "bf16"), (128, 512, 8, 8, 256, "bf16"),
                                             (1, 256, 4, 1, 272, "f16"), (37, 4096, 8, 2, 2048, "f16")])
def test_dense_gate_up_matches_the_routed_projection(F, T, H, E, k, N, dtype):
    """The gate/up projection computed from the un-permuted tokens (every expert against all
    tokens, the routing applied in the epilogue) against the routed grouped GEMM on the
    gathered rows and against the oracle; one expert is left without tokens."""
    from ppl.pmx_b200.torch_function.moe import moe_grouped_linear, grouped_linear_check
    rng = np.random.default_rng(T + N)
    x = orc.round_to_dtype(rng.standard_normal((T, H)).astype(np.float32), dtype)
    sc = rng.standard_normal((T, E)).astype(np.float32)
    if E > k:
        sc[:, E // 2] = -1e4                       # nobody picks this expert
    sc, _ = orc.detie_scores(sc, dtype)
    w = orc.round_to_dtype((rng.standard_normal((E, N, H)) / np.sqrt(H)).astype(np.float32), dtype)
    b = orc.round_to_dtype(rng.standard_normal((E, N)).astype(np.float32), dtype)
    xd, wd, bd = dev(x, dtype), dev(w, dtype), dev(b, dtype)
    xe, ew, inv, off = F.moe_select(xd, dev(sc, dtype), E, k)
    for bias in (None, bd):
        h, ws = F.moe_dense_gate_up(xd, inv, off, wd, bias, return_workspace=True)
        grouped_linear_check(ws)
        routed = moe_grouped_linear(xe.view(-1, H), off, wd, bias, swiglu=True, zero_outside=False)
        oxe, _, _, ooff = orc.moe_select(x, sc, E, k, dtype)
        ref = orc.swiglu(orc.moe_grouped_linear(oxe, ooff, w, None if bias is None else b))
        assert_close(h, ref, dtype)
        assert_close(h, host(routed), dtype)
    assert h.shape == (T * k, N // 2)


@pytest.mark.parametrize("T,H,E,k,N,dtype", [(64, 512, 8, 2, 1024, "f16"), (16, 256, 8, 2, 3584, "f16"),
                                             (33, 1024, 4, 2, 784, "bf16"), (64, 4096, 8, 2, 3584, "f16"),
                                             (1, 256, 4, 1, 272, "f16"), (48, 328, 16, 4, 528, "bf16"),
                                             (64, 2048, 8, 8, 512, "bf16"), (128, 1024, 8, 2, 768, "f16"),
                                             (100, 512, 4, 2, 528, "bf16")])
def test_dense_mlp_matches_two_launches_and_the_oracle(F, T, H, E, k, N, dtype):
    """Both expert projections in one launch against the oracle, against the dense gate/up
    launch followed by the routed down projection, and against itself when launches follow
    each other directly on the stream (each must see the counters of its own launch only);
    one expert is left without tokens, H and N/2 need not be multiples of the tile sizes."""
    from ppl.pmx_b200.torch_function.moe import moe_grouped_linear, dense_mlp_check
    rng = np.random.default_rng(T + N + H)
    x = orc.round_to_dtype(rng.standard_normal((T, H)).astype(np.float32), dtype)
    sc = rng.standard_normal((T, E)).astype(np.float32)
    if E > k:
        sc[:, E // 2] = -1e4                       # nobody picks this expert
    sc, _ = orc.detie_scores(sc, dtype)
    wu = orc.round_to_dtype((rng.standard_normal((E, N, H)) / np.sqrt(H)).astype(np.float32), dtype)
    w2 = orc.round_to_dtype((rng.standard_normal((E, H, N // 2)) / np.sqrt(N // 2)).astype(np.float32), dtype)
    xd, wud, w2d = dev(x, dtype), dev(wu, dtype), dev(w2, dtype)
    _, ew, inv, off = F.moe_select(xd, dev(sc, dtype), E, k)
    y, ws = F.moe_dense_mlp(xd, inv, off, wud, w2d, return_workspace=True)
    dense_mlp_check(ws, E)
    assert y.shape == (T * k, H)
    assert int(ws[256:256 + 4 * (E + 1)].view(torch.int32).abs().sum()) == 0, "the counters must be left zero"
    h = F.moe_dense_gate_up(xd, inv, off, wud, None)
    two = moe_grouped_linear(h, off, w2d, None, zero_outside=False)
    oxe, _, _, ooff = orc.moe_select(x, sc, E, k, dtype)
    oh = orc.round_to_dtype(orc.swiglu(orc.moe_grouped_linear(oxe, ooff, wu, None)), dtype)
    ref = orc.moe_grouped_linear(oh, ooff, w2, None)
    assert_close(y, ref, dtype)
    assert_close(y, host(two), dtype)
    # launches directly behind one another
    ys = [F.moe_dense_mlp(xd, inv, off, wud, w2d) for _ in range(4)]
    torch.cuda.synchronize()
    dense_mlp_check(ws, E)
    for other in ys:
        assert torch.equal(other, y)


def test_block_one_launch_experts_equals_two_launches(F):
    """MoeFeedForward with both expert projections in one launch against the same block with
    the dense gate/up launch + the down launch, eagerly and replayed from a CUDA graph."""
    from ppl.pmx_b200 import workloads as W
    from ppl.pmx_b200.moe_layers import MoeFeedForward
    from ppl.pmx_b200.torch_function.moe import dense_mlp_covers
    sh = W.scaled(W.WORKLOADS["decode_t64"], H=1024, I=1792)
    x, wr, _, _ = W.make_activations(sh)
    wu, w2 = W.make_expert_weights(sh, "cuda")
    assert dense_mlp_covers(sh.T, wu, w2, sh.k), "this shape must take the one-launch path"
    blocks = []
    for one in (True, False):
        blk = MoeFeedForward(sh.H, sh.I, sh.E, sh.k, None, False, one_launch_experts=one).cuda().half()
        with torch.no_grad():
            blk.gate.weight.copy_(wr)
            blk.wu.weight.copy_(wu)
            blk.w2.weight.copy_(w2)
        blocks.append(blk)
    xd = x.cuda()
    with torch.no_grad():
        a, b = blocks[0](xd), blocks[1](xd)
        torch.cuda.synchronize()
        blocks[0].check()
        assert blocks[0]._mlp_ws is not None and blocks[1]._mlp_ws is None
        torch.testing.assert_close(a.float(), b.float(), atol=2e-3, rtol=2e-3)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            blocks[0](xd)
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = blocks[0](xd)
        for _ in range(20):
            g.replay()
        torch.cuda.synchronize()
        blocks[0].check()
        assert torch.equal(out, a)
        g.reset()


def test_weight_prefetch_ahead_of_the_wait_gives_the_same_result(F):
    """The optional request of the first item's weight tiles before the dependency wait
    (pmx_moe_set_weight_prefetch, off by default), with a right guess (every expert owns
    rows) and a wrong one (an empty expert): bit-identical to the plain path."""
    from ppl.pmx_b200._cabi import lib, GemmPlan
    from ppl.pmx_b200.torch_function.moe import moe_grouped_linear
    rng = np.random.default_rng(77)
    M, N, K, E = 96, 512, 1024, 8
    x = dev(rng.standard_normal((M, K)).astype(np.float32), "f16")
    w = dev((rng.standard_normal((E, N, K)) / np.sqrt(K)).astype(np.float32), "f16")
    for empty in (0, 2):
        off = torch.from_numpy(ragged_offsets(rng, M, E, empty=empty)).cuda()
        plain = moe_grouped_linear(x, off, w, None, plan=GemmPlan(kernel=2))
        old = lib.pmx_moe_set_weight_prefetch(1)
        try:
            ahead = moe_grouped_linear(x, off, w, None, plan=GemmPlan(kernel=2))
            torch.cuda.synchronize()
        finally:
            lib.pmx_moe_set_weight_prefetch(old)
        assert torch.equal(plain, ahead)


def test_tuning_switches_do_not_change_results_and_stamps_are_recorded(F):
    """The L2 prefetch distance, the rows per gate/up item of the one-launch kernel and the
    time stamps are diagnostics / tuning: same bits with any setting; a launch made while a
    stamp buffer is set leaves increasing %globaltimer values in its slot."""
    import ctypes as C
    from ppl.pmx_b200._cabi import lib
    from ppl.pmx_b200.torch_function.moe import moe_grouped_linear
    rng = np.random.default_rng(5)
    T, H, E, k, N = 32, 512, 8, 2, 768
    x = dev(rng.standard_normal((T, H)).astype(np.float32), "f16")
    sc, _ = orc.detie_scores(rng.standard_normal((T, E)).astype(np.float32), "f16")
    wu = dev((rng.standard_normal((E, N, H)) / np.sqrt(H)).astype(np.float32), "f16")
    w2 = dev((rng.standard_normal((E, H, N // 2)) / np.sqrt(N // 2)).astype(np.float32), "f16")
    xe, ew, inv, off = F.moe_select(x, dev(sc, "f16"), E, k)
    base_y = F.moe_dense_mlp(x, inv, off, wu, w2)
    base_h = moe_grouped_linear(xe.view(-1, H), off, wu, None, swiglu=True, zero_outside=False)
    old = lib.pmx_moe_set_l2_prefetch(4)
    try:
        assert torch.equal(F.moe_dense_mlp(x, inv, off, wu, w2), base_y)
        assert torch.equal(moe_grouped_linear(xe.view(-1, H), off, wu, None, swiglu=True, zero_outside=False), base_h)
    finally:
        lib.pmx_moe_set_l2_prefetch(old)
    for rows in (64, 96, 128):
        lib.pmx_moe_dense_mlp_set_rows(rows)
        try:
            assert torch.equal(F.moe_dense_mlp(x, inv, off, wu, w2), base_y)
        finally:
            lib.pmx_moe_dense_mlp_set_rows(0)
    buf = torch.zeros(4 * 160 * 8, dtype=torch.int64, device="cuda")
    assert lib.pmx_moe_set_stamp_buffer(C.c_void_p(buf.data_ptr()), buf.numel() * 8) == 4
    try:
        y = F.moe_dense_mlp(x, inv, off, wu, w2)
        torch.cuda.synchronize()
        ids = (C.c_int32 * 8)()
        assert lib.pmx_moe_stamp_slots(ids, 8) == 1 and ids[0] == 4
    finally:
        lib.pmx_moe_set_stamp_buffer(None, 0)
    assert torch.equal(y, base_y)
    s = buf.view(4, 160, 8)[0].cpu().numpy()
    active = s[:, 0] > 0
    assert active.sum() >= 1
    assert (s[active, 6] >= s[active, 1]).all() and (s[active, 1] >= s[active, 0]).all()


def test_block_dense_decode_path_equals_the_routed_path(F):
    """MoeFeedForward with the router + dense gate/up path (decode-size batch) against the
    same block with that path switched off, eagerly and replayed from a CUDA graph."""
    from ppl.pmx_b200 import workloads as W
    from ppl.pmx_b200.moe_layers import MoeFeedForward
    from ppl.pmx_b200.torch_function.moe import dense_gate_up_covers
    sh = W.scaled(W.WORKLOADS["decode_t64"], H=512, I=1024)
    x, wr, _, _ = W.make_activations(sh)
    wu, w2 = W.make_expert_weights(sh, "cuda")
    assert dense_gate_up_covers(sh.T, wu, sh.k), "this shape must take the dense path"
    assert not dense_gate_up_covers(128, wu, sh.k) and not dense_gate_up_covers(4, wu, sh.k)
    blocks = []
    for dense in (True, False):
        blk = MoeFeedForward(sh.H, sh.I, sh.E, sh.k, None, False, dense_decode=dense).cuda().half()
        with torch.no_grad():
            blk.gate.weight.copy_(wr)
            blk.wu.weight.copy_(wu)
            blk.w2.weight.copy_(w2)
        blocks.append(blk)
    xd = x.cuda()
    with torch.no_grad():
        a, b = blocks[0](xd), blocks[1](xd)
        torch.cuda.synchronize()
        blocks[0].check()
        torch.testing.assert_close(a.float(), b.float(), atol=2e-3, rtol=2e-3)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            blocks[0](xd)
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = blocks[0](xd)
        for _ in range(5):
            g.replay()
        torch.cuda.synchronize()
        torch.testing.assert_close(out.float(), b.float(), atol=2e-3, rtol=2e-3)
        g.reset()


def test_grouped_linear_auto_plan_and_fp32(F):
    rng = np.random.default_rng(12)
    run_linear(F, rng, 4500, 256, 128, 4, "bf16", bias=True)   # auto -> paired CTAs (>= 1024 rows per expert)
    run_linear(F, rng, 4500, 512, 128, 4, "bf16", swiglu=True)
    run_linear(F, rng, 700, 256, 128, 4, "f16")          # auto -> tokens on M
    run_linear(F, rng, 24, 256, 1024, 8, "f16")          # auto -> weights on M (+ split-K)
    run_linear(F, rng, 50, 100, 36, 4, "f16")            # N, K not multiples of 8 -> CUDA-core kernel
    run_linear(F, rng, 130, 96, 200, 6, "f32", bias=True)
    run_linear(F, rng, 130, 96, 200, 6, "f32", swiglu=True)


@pytest.mark.parametrize("M,N,K,dtype", [(64, 4096, 4096, "f16"), (1, 6144, 4096, "f16"), (300, 520, 192, "bf16"),
                                         # the router gate of a decode batch through `linear`: few output
                                         # features, long K (K is sliced)
                                         (64, 8, 4096, "f16"), (16, 64, 2048, "bf16"), (128, 8, 14336, "f16"),
                                         (4096, 8, 4096, "bf16"), (2500, 64, 2048, "f16"), (3000, 1024, 512, "bf16"),
                                         (70, 100, 36, "f16"), (33, 96, 200, "f32")])
def test_dense_linears(F, M, N, K, dtype):
    """linear / column_parallel_linear / row_parallel_linear without a process group (the
    grouped kernel with one expert and no offset table) against the oracle's matrix product:
    attention projections at decode and prefill sizes, the router gate for large batches
    (N = 8 and 64), odd shapes and fp32 on the CUDA-core kernel."""
    rng = np.random.default_rng(M + N + K)
    x = orc.round_to_dtype(rng.standard_normal((M, K)).astype(np.float32), dtype)
    w = orc.round_to_dtype((rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32), dtype)
    b = orc.round_to_dtype(rng.standard_normal(N).astype(np.float32), dtype)
    ref = orc.moe_grouped_linear(x, np.array([0, M]), w[None], None)
    xd, wd, bd = dev(x, dtype), dev(w, dtype), dev(b, dtype)
    assert_close(F.linear(xd, wd, None, K, N), ref, dtype)
    assert_close(F.linear(xd.view(1, M, K), wd, bd, K, N).view(M, N), ref + b, dtype)
    assert_close(F.column_parallel_linear(xd, wd, bd, None, K, N, True), ref + b, dtype)
    assert_close(F.row_parallel_linear(xd, wd, bd, None, K, N, True), ref + b, dtype)
    assert_close(F.router_gate(xd, wd), ref, dtype)
    with pytest.raises(Exception):
        F.row_parallel_linear(xd, wd, None, None, K, N, False)      # the reference raises too


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_dense_linear_golden(F, dtype):
    """Golden vectors of the reference's linear / column_parallel_linear / row_parallel_linear
    (run on CPU without a process group)."""
    g = load(f"dense_linear_{dtype}.npz")
    x, w, b = dev(g["x"], dtype), dev(g["w"], dtype), dev(g["b"], dtype)
    K, N = w.shape[1], w.shape[0]
    assert_close(F.linear(x, w, None, K, N), g["linear"], dtype)
    assert_close(F.linear(x, w, b, K, N), g["linear_bias"], dtype)
    assert_close(F.column_parallel_linear(x, w, b, None, K, N, True), g["column"], dtype)
    assert_close(F.row_parallel_linear(x, w, b, None, K, N, True), g["row"], dtype)
    assert_close(F.linear(x, w, b, K, N), g["linear_bias_fp32"], dtype)


def test_grouped_linear_errors(F):
    x = torch.randn(8, 64, device="cuda", dtype=torch.float16)
    w = torch.randn(4, 32, 64, device="cuda", dtype=torch.float16)
    off = torch.tensor([0, 2, 4, 6, 8])
    with pytest.raises(AssertionError):
        F.moe_column_parallel_linear(x, off, w, None, None, 4, 32, 32, False)   # in_features mismatch
    with pytest.raises(ValueError):
        F.moe_column_parallel_linear(x, off[:4], w, None, None, 4, 64, 32, False)
    with pytest.raises(TypeError):
        F.moe_column_parallel_linear(x, off, w.float(), None, None, 4, 64, 32, False)
    with pytest.raises(RuntimeError):
        F.moe_row_parallel_linear(x.cpu(), off, w.cpu(), None, None, 4, 64, 32, True)


# --------------------------------------------------------------------------- reduce
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_reduce_golden(F, dtype):
    g = load(f"reduce_{dtype}.npz")
    out = F.moe_reduce(dev(g["y"], dtype), dev(g["expert_weights"], dtype),
                       torch.from_numpy(g["invert_permutation"]).cuda(), int(g["k"]))
    assert_close(out, g["out"], dtype)
    ref = orc.moe_reduce(g["y"].reshape(-1, g["y"].shape[-1]), g["expert_weights"], g["invert_permutation"], int(g["k"]))
    assert_close(out, ref, dtype)


@pytest.mark.parametrize("T,k,N,dtype", [(1, 2, 4096, "f16"), (300, 8, 2048, "bf16"), (33, 3, 50, "f16"), (64, 2, 72, "f32")])
def test_reduce_shapes(F, T, k, N, dtype):
    rng = np.random.default_rng(T)
    y = orc.round_to_dtype(rng.standard_normal((T * k, N)).astype(np.float32), dtype)
    w = orc.round_to_dtype(rng.random((T, k)).astype(np.float32), dtype)
    inv = rng.permutation(T * k).reshape(T, k)
    out = F.moe_reduce(dev(y, dtype).view(T, k, N), dev(w, dtype), torch.from_numpy(inv).cuda(), k)
    assert out.shape == (T, N)
    assert_close(out, orc.moe_reduce(y, w, inv, k), dtype)


def test_reduce_allreduce_kernel_with_a_single_rank(F):
    """The fused combine + all-reduce kernel with world = 1 (its exchange buffer is then
    just local memory): same result as moe_reduce, on consecutive calls that alternate
    between the two exchange algorithms."""
    import ctypes as C
    from ppl.pmx_b200._cabi import lib, check, ptr, stream_of
    T, k, N = 70, 2, 512
    nbytes = lib.pmx_moe_reduce_allreduce_buffer_bytes(T, N, 0)
    buf = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    table = (C.c_void_p * 1)(buf.data_ptr())
    for call in range(3):
        rng = np.random.default_rng(call)
        y = orc.round_to_dtype(rng.standard_normal((T * k, N)).astype(np.float32), "f16")
        w = orc.round_to_dtype(rng.random((T, k)).astype(np.float32), "f16")
        inv = rng.permutation(T * k).reshape(T, k)
        out = torch.empty(T, N, dtype=torch.float16, device="cuda")
        yd, wd, invd = dev(y, "f16"), dev(w, "f16"), torch.from_numpy(inv).cuda()
        check(lib.pmx_moe_reduce_allreduce(ptr(yd), ptr(wd), ptr(invd), ptr(out), T, k, N, 0, table, 0, 1,
                                           nbytes, 1 + call % 2, 0, 0, stream_of(out)))
        rec = (C.c_int32 * 4)()
        check(lib.pmx_moe_reduce_allreduce_check(ptr(buf), C.byref(rec), stream_of(out)))
        assert_close(out, orc.moe_reduce(y, w, inv, k), "f16")
        assert torch.equal(out, F.moe_reduce(yd.view(T, k, N), wd, invd, k))


def _emulated_allreduce(world, algo, T_seq, N=512, k=2, dtype="f16", T_max=None):
    """All `world` ranks of the exchange as one cooperative launch on this GPU; returns
    nothing, asserts every rank's result against the oracle and against each other."""
    import ctypes as C
    from ppl.pmx_b200._cabi import lib, check, ptr, DTYPE_CODE
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[dtype]
    code = DTYPE_CODE[tdt]
    nbytes = lib.pmx_moe_reduce_allreduce_buffer_bytes(T_max or max(T_seq), N, code)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    table = (C.c_void_p * world)(*[b.data_ptr() for b in bufs])
    arr = lambda ts: (C.c_void_p * world)(*[t.data_ptr() for t in ts])
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, T in enumerate(T_seq):
        rng = np.random.default_rng(100 * world + call)
        w = orc.round_to_dtype(rng.random((T, k)).astype(np.float32), dtype)
        inv = rng.permutation(T * k).reshape(T, k)
        ys = [orc.round_to_dtype(rng.standard_normal((T * k, N)).astype(np.float32), dtype) for _ in range(world)]
        yd = [dev(y, dtype) for y in ys]
        wd = [dev(w, dtype) for _ in range(world)]
        invd = [torch.from_numpy(inv).cuda() for _ in range(world)]
        outs = [torch.full((T, N), float("nan"), dtype=tdt, device="cuda") for _ in range(world)]
        check(lib.pmx_moe_reduce_allreduce_emulated(arr(yd), arr(wd), arr(invd), arr(outs), T, k, N, code, table, world,
                                                    nbytes, algo, 0, stream))
        rec = (C.c_int32 * 4)()
        for b in bufs:
            check(lib.pmx_moe_reduce_allreduce_check(ptr(b), C.byref(rec), stream))
        # partial results are rounded to the tensor type before they are exchanged
        ref = sum(orc.round_to_dtype(orc.moe_reduce(y, w, inv, k), dtype) for y in ys)
        for r in range(world):
            assert_close(outs[r], ref, dtype, f"world={world} algo={algo} call={call} T={T} rank={r}")
            assert torch.equal(outs[r], outs[0]), "ranks must hold bit-identical sums"


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("algo", [1, 2])
def test_reduce_allreduce_protocol_with_emulated_ranks(F, world, algo):
    """The multi-rank exchange protocols (flags, epochs, slot reuse, changing T on one
    set of buffers) with every rank played by one slice of a single cooperative launch."""
    _emulated_allreduce(world, algo, [64, 8, 64, 8, 1, 70, 70], T_max=70)
    _emulated_allreduce(world, algo, [33, 5], N=2048, dtype="bf16")
    _emulated_allreduce(world, algo, [9, 9], N=64, k=3, dtype="f32")


@pytest.mark.parametrize("algo", [1, 2])
def test_reduce_allreduce_wait_runs_out_and_is_reported(F, algo):
    """Failure detection without a fault: rank 0 of a 2-rank group runs alone, so its
    waits on rank 1 (whose buffer nobody writes) run out after the 20 ms limit.  The kernel
    returns, the check reports who was missing, the rows it could not finish are zero,
    and after clearing the buffers the next exchange works."""
    import ctypes as C
    from ppl.pmx_b200._cabi import lib, check, ptr, stream_of, PmxError
    T, k, N = 16, 2, 512
    nbytes = lib.pmx_moe_reduce_allreduce_buffer_bytes(T, N, 0)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    table = (C.c_void_p * 2)(*[b.data_ptr() for b in bufs])
    rng = np.random.default_rng(0)
    y = dev(rng.standard_normal((T * k, N)).astype(np.float32), "f16")
    w = dev(rng.random((T, k)).astype(np.float32), "f16")
    inv = torch.from_numpy(rng.permutation(T * k).reshape(T, k)).cuda()
    out = torch.full((T, N), float("nan"), dtype=torch.float16, device="cuda")
    check(lib.pmx_moe_reduce_allreduce(ptr(y), ptr(w), ptr(inv), ptr(out), T, k, N, 0, table, 0, 2, nbytes, algo, 0,
                                       20_000_000, stream_of(out)))
    rec = (C.c_int32 * 4)()
    status = lib.pmx_moe_reduce_allreduce_check(ptr(bufs[0]), C.byref(rec), stream_of(out))
    assert status == -6 and rec[0] == 1 and rec[1] == 1, (status, list(rec))
    assert b"waiting for rank 1" in lib.pmx_moe_last_error()
    assert not torch.isnan(out).any(), "every row must hold a defined value after a timeout"
    assert (out == 0).any()
    # the record is cleared by the check; fresh buffers -> the next exchange is clean
    assert lib.pmx_moe_reduce_allreduce_check(ptr(bufs[0]), C.byref(rec), stream_of(out)) == 0
    for b in bufs:
        b.zero_()
    one = (C.c_void_p * 1)(bufs[0].data_ptr())
    check(lib.pmx_moe_reduce_allreduce(ptr(y), ptr(w), ptr(inv), ptr(out), T, k, N, 0, one, 0, 1, nbytes, algo, 0,
                                       20_000_000, stream_of(out)))
    check(lib.pmx_moe_reduce_allreduce_check(ptr(bufs[0]), C.byref(rec), stream_of(out)))
    assert torch.equal(out, F.moe_reduce(y.view(T, k, N), w, inv, k))


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_rms_norm_golden(F, dtype):
    g = load(f"rmsnorm_{dtype}.npz")
    ulp = 1.5 * {"f32": 2.0 ** -22, "f16": 2.0 ** -9, "bf16": 2.0 ** -6}[dtype]   # 3 ulp: rsqrt + two roundings
    x, sk, w = dev(g["x"], dtype), dev(g["skip"], dtype), dev(g["weight"], dtype)
    y, s = F.skip_rms_norm(x, w, sk, -1, 1e-5)
    assert y.shape == x.shape and s.shape == x.shape and y.dtype == x.dtype
    assert np.array_equal(host(s), g["skip_out"])                       # the residual stream is bit-exact
    np.testing.assert_allclose(host(y), g["y_skip"], rtol=ulp, atol=1e-6)
    y, s = F.skip_rms_norm(x, w, None, -1, 1e-6)
    assert s is x or torch.equal(s, x)
    np.testing.assert_allclose(host(y), g["y_noskip"], rtol=ulp, atol=1e-6)
    np.testing.assert_allclose(host(F.rms_norm(x, w, -1, 1e-5)), g["y_plain"], rtol=ulp, atol=1e-6)
    oy, _ = orc.skip_rms_norm(g["x"], g["weight"], g["skip"], 1e-5, dtype)
    np.testing.assert_allclose(host(F.skip_rms_norm(x, w, sk)[0]), oy, rtol=ulp, atol=1e-6)


@pytest.mark.parametrize("M,H,dtype", [(1, 4096, "f16"), (64, 4096, "f16"), (300, 1000, "bf16"), (7, 50, "f32"), (2000, 2048, "bf16"),
                                       # many rows: the warp-per-row kernel (rows of up to 512 sixteen-byte chunks)
                                       (3000, 4096, "f16"), (2500, 1000, "bf16"), (2100, 2048, "f32"), (2049, 8, "f16")])
def test_rms_norm_shapes(F, M, H, dtype):
    rng = np.random.default_rng(M + H)
    x = orc.round_to_dtype(rng.standard_normal((M, H)).astype(np.float32) * 3, dtype)
    sk = orc.round_to_dtype(rng.standard_normal((M, H)).astype(np.float32), dtype)
    w = orc.round_to_dtype(1 + 0.2 * rng.standard_normal(H).astype(np.float32), dtype)
    ulp = 1.5 * {"f32": 2.0 ** -22, "f16": 2.0 ** -9, "bf16": 2.0 ** -6}[dtype]   # 3 ulp: rsqrt + two roundings
    y, s = F.skip_rms_norm(dev(x, dtype), dev(w, dtype), dev(sk, dtype), -1, 1e-5)
    oy, os_ = orc.skip_rms_norm(x, w, sk, 1e-5, dtype)
    assert np.array_equal(host(s), os_)
    np.testing.assert_allclose(host(y), oy, rtol=ulp, atol=1e-6)
    oy2, _ = orc.skip_rms_norm(x, w, None, 1e-5, dtype)
    np.testing.assert_allclose(host(F.rms_norm(dev(x, dtype), dev(w, dtype), -1, 1e-5)), oy2, rtol=ulp, atol=1e-6)
    with pytest.raises(ValueError):
        F.rms_norm(dev(x, dtype), dev(w, dtype), 0)
    with pytest.raises(RuntimeError):
        F.rms_norm(dev(x, dtype).cpu(), dev(w, dtype).cpu())


# --------------------------------------------------------------------------- block
@pytest.mark.parametrize("name", ["block_f32", "block_f16", "block_bf16", "block_f16_fine"])
@pytest.mark.parametrize("fused", [False, True])
def test_block_golden(F, name, fused):
    from ppl.pmx_b200.moe_layers import MoeFeedForward
    g = load(name + ".npz")
    dtype, E, k = str(g["dtype"]), int(g["E"]), int(g["k"])
    H, I = g["x"].shape[-1], g["w_down"].shape[-1]
    blk = MoeFeedForward(H, I, E, k, None, False, fused=fused).cuda().to(dev(g["x"], dtype).dtype)
    with torch.no_grad():
        blk.gate.weight.copy_(dev(g["w_router"], dtype))
        blk.wu.weight.copy_(dev(g["w_gate_up"], dtype))
        blk.w2.weight.copy_(dev(g["w_down"], dtype))
        out = blk(dev(g["x"], dtype), router_logits=dev(g["scores"], dtype))
    assert_close(out, g["out_fp32_reference"], dtype, "vs fp32 run of the reference ops")
    assert_close(out, g["out"], dtype, "vs low-precision run of the reference ops")
    r = orc.moe_block(g["x"], g["w_router"], g["w_gate_up"], g["w_down"], E, k, dtype, scores=g["scores"],
                      round_intermediates=False)
    assert_close(out, r["out"], dtype, "vs oracle")


def test_block_with_its_own_router(F):
    """MoeFeedForward computing the router logits itself (fused router + select for a
    decode-size batch, the dense-linear kernel + moe_select for a large one) against the
    oracle fed with the scores the block produced."""
    from ppl.pmx_b200 import workloads as W
    from ppl.pmx_b200.moe_layers import MoeFeedForward
    for wl, kw in (("decode_t64", dict(H=512, I=1024)), ("prefill", dict(T=1500, H=256, I=512))):
        sh = W.scaled(W.WORKLOADS[wl], **kw)
        x, wr, _, _ = W.make_activations(sh)
        wu, w2 = W.make_expert_weights(sh, "cuda")
        blk = MoeFeedForward(sh.H, sh.I, sh.E, sh.k, None, False).cuda().to(W.TORCH_DTYPE[sh.dtype])
        with torch.no_grad():
            blk.gate.weight.copy_(wr)
            blk.wu.weight.copy_(wu)
            blk.w2.weight.copy_(w2)
            out = blk(x.cuda())
            routed = F.moe_route_select(x.cuda(), blk.gate.weight, sh.E, sh.k)
            sc = routed[0] if routed is not None else F.router_gate(x.cuda(), blk.gate.weight)
        r = orc.moe_block(host(x), host(wr), host(wu), host(w2), sh.E, sh.k, sh.dtype, scores=host(sc),
                          round_intermediates=False)
        assert_close(out, r["out"], sh.dtype, wl)


@pytest.mark.parametrize("wl,scale", [("decode_t64", 8), ("prefill", 16), ("finegrained_empty", 4)])
def test_block_scaled_workloads(F, wl, scale):
    """The measured workloads with H and I divided by `scale` (T, E, k and the
    router statistics kept), end to end against the oracle."""
    from ppl.pmx_b200 import workloads as W
    from ppl.pmx_b200.moe_layers import MoeFeedForward
    sh = W.WORKLOADS[wl]
    sh = W.scaled(sh, H=sh.H // scale, I=sh.I // scale, T=min(sh.T, 1024))
    x, wr, sc, _ = W.make_activations(sh)
    wu, w2 = W.make_expert_weights(sh, "cuda")
    blk = MoeFeedForward(sh.H, sh.I, sh.E, sh.k, None, False).cuda().to(W.TORCH_DTYPE[sh.dtype])
    with torch.no_grad():
        blk.wu.weight.copy_(wu)
        blk.w2.weight.copy_(w2)
        out = blk(x.cuda(), router_logits=sc.cuda())
    r = orc.moe_block(host(x), host(wr), host(wu), host(w2), sh.E, sh.k, sh.dtype, scores=host(sc),
                      round_intermediates=False)
    assert_close(out, r["out"], sh.dtype)


@pytest.mark.parametrize("H,I,T", [(512, 1024, 48), (4096, 1792, 64)])      # toy width; a rank's shard of Mixtral at tp 8
@pytest.mark.parametrize("fused_ffn_glu", [True, False])
def test_reference_moe_block_runs_on_the_patched_operators(F, fused_ffn_glu, H, I, T):
    """The drop-in claim itself: the reference's own MoeFeedForward module
    (model_zoo/mixtral/modeling/dynamic_batching/Model.py:155-214, unmodified, staged under
    oracle/_ref) is built, the operators are swapped in with patch_reference(), and its
    output must match the oracle (fp32 math on the same routing)."""
    import oracle
    if oracle.ref_path() is None:
        pytest.skip("the OPMX reference is not staged (python oracle/make_ref.py)")
    from ppl.pmx_b200 import workloads as W
    from ppl.pmx_b200.moe_layers import patch_reference, unpatch_reference
    opmx, model, ModelParams = oracle.import_reference_mixtral()
    sh = W.scaled(W.WORKLOADS["decode_t64"], H=H, I=I, T=T)
    x, wr, _, _ = W.make_activations(sh)
    wu, w2 = W.make_expert_weights(sh, "cuda")
    params = ModelParams(hidden_dim=sh.H, intermediate_dim=sh.I, num_experts=sh.E, num_experts_per_token=sh.k)
    blk = model.MoeFeedForward(params, 0, fused_ffn_glu, False, None).cuda().half()
    with torch.no_grad():
        blk.gate.weight.copy_(wr)
        if fused_ffn_glu:
            blk.wu.weight.copy_(wu)
        else:
            blk.w1.weight.copy_(wu[:, :sh.I])
            blk.w3.weight.copy_(wu[:, sh.I:])
        blk.w2.weight.copy_(w2)
    saved = patch_reference(opmx)
    try:
        with torch.no_grad():
            out = blk(x.cuda())
            sc = F.linear(x.cuda(), blk.gate.weight, None, sh.H, sh.E)
    finally:
        unpatch_reference(opmx, saved)
    assert_close(sc, orc.linear(host(x), host(wr)), sh.dtype, "router logits")
    r = orc.moe_block(host(x), host(wr), host(wu), host(w2), sh.E, sh.k, sh.dtype, scores=host(sc),
                      round_intermediates=False)
    assert_close(out, r["out"], sh.dtype)
    # and against the unmodified reference operators on the same GPU (its linears allocate with the
    # global default dtype and device, so it runs under the regime its loader sets)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.float16)
    torch.set_default_device("cuda")
    try:
        with torch.no_grad():
            ref_out = blk(x.cuda())
    finally:
        torch.set_default_device("cpu")
        torch.set_default_dtype(old)
    # the reference routes on cuBLAS logits: tokens whose two best logits are within rounding of
    # each other may pick another expert there, so compare the bulk of the tokens
    close = ((out.float() - ref_out.float()).abs() <= 2e-2 + 1e-2 * ref_out.float().abs()).all(dim=-1)
    assert close.float().mean() >= 0.9, f"only {int(close.sum())} of {T} tokens agree with the reference operators"
