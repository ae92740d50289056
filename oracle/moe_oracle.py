"""CPU oracle for the OPMX mixture-of-experts path.  TEST INFRASTRUCTURE ONLY.

This module is the checker the CUDA path is compared against.  It is imported
by the test-suite, by the smoke test and by the CPU-baseline leg of the
benchmark; the product package never imports it and has no CPU fallback.

Each function restates, in numpy, what the corresponding OPMX reference
operator computes (file:line given per function, relative to the OPMX tree).
Floating-point work is carried out in float32 (float64 accumulation for the
matrix products) on exact up-casts of the low-precision inputs, which is the
"reference computed in fp32" the parity tolerance (max-abs 2e-2 / rel 1e-2) is
stated against.  Integer results (expert ids, expert_offset,
invert_permutation) are exact.

Parity pin: the reference ships no golden vectors, so this restatement is
pinned against outputs of the reference operators themselves, run on CPU from
the OPMX tree and stored under tests/golden/ by tests/golden/make_golden.py.

Tie rule.  `torch.topk` leaves the order of equal scores implementation
defined.  The oracle (and the CUDA kernel) use: higher score first, lower
expert index first among equal scores, NaN ranks above every number.  On rows
without equal scores inside the top-(k+1) this is exactly torch's result.
"""
from __future__ import annotations

import numpy as np

__all__ = [
    "bf16_bits_to_f32", "f32_to_bf16_bits", "round_to_dtype", "topk_desc",
    "moe_select", "moe_grouped_linear", "swiglu", "silu_gate", "moe_reduce",
    "moe_block", "detie_scores", "rows_with_ties", "skip_rms_norm", "linear", "decode_cache_attention",
    "cache_view",
]


# ----------------------------------------------------------------------------
# dtype helpers (numpy has no bfloat16: it is carried as uint16 bit patterns)
# ----------------------------------------------------------------------------
def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """Exact up-cast of bfloat16 bit patterns (uint16) to float32."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round float32 to bfloat16 (round-to-nearest-even), returned as uint16."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = np.isnan(x)
    rounded = (u + (0x7FFF + ((u >> 16) & 1))) >> 16
    rounded = np.where(nan, 0x7FC0, rounded)
    return rounded.astype(np.uint16)


def round_to_dtype(x: np.ndarray, dtype: str) -> np.ndarray:
    """Round a float32 array once to `dtype` ("f32" | "f16" | "bf16") and
    return the rounded values as float32."""
    x = np.asarray(x, dtype=np.float32)
    if dtype == "f32":
        return x
    if dtype == "f16":
        return x.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        return bf16_bits_to_f32(f32_to_bf16_bits(x))
    raise ValueError(f"unknown dtype {dtype!r}")


# ----------------------------------------------------------------------------
# routing
# ----------------------------------------------------------------------------
def _order_key(scores: np.ndarray) -> np.ndarray:
    """Map float32 scores to uint32 keys whose unsigned order is the score
    order used by the routing rule: -0 == +0, NaN above +inf."""
    s = np.ascontiguousarray(scores, dtype=np.float32)
    s = np.where(s == 0.0, np.float32(0.0), s)          # -0 -> +0
    u = s.view(np.uint32)
    key = np.where(u >> 31 == 1, ~u, u | np.uint32(0x80000000)).astype(np.uint32)
    return np.where(np.isnan(s), np.uint32(0xFFFFFFFF), key)


def topk_desc(scores: np.ndarray, k: int):
    """Top-k per row, descending, ties -> lower index.  Follows
    torch_function/MoeSelect.py:40 (`torch.topk(scores, k, dim=-1)`, sorted)
    with the tie rule stated in the module docstring.
    Returns (values float32 [T,k], indices int64 [T,k])."""
    s = np.asarray(scores, dtype=np.float32)
    T, E = s.shape
    if not 0 < k <= E:
        raise ValueError("k out of range")
    key = _order_key(s).astype(np.int64)
    # stable argsort of the negated key: descending score, ascending index
    order = np.argsort(-key, axis=1, kind="stable")[:, :k]
    vals = np.take_along_axis(s, order, axis=1)
    return vals, order.astype(np.int64)


def moe_select(x: np.ndarray, scores: np.ndarray, num_experts: int, k: int,
               dtype: str = "f32"):
    """torch_function/MoeSelect.py:36-64.

    x: [T,H] float32 (exact up-cast of the activation dtype), scores: [T,E]
    float32 (exact up-cast).  Returns
      x_expand_permute [T*k,H] float32   (MoeSelect.py:45-47)
      expert_weights   [T,k]   float32, rounded once to `dtype` (:40-41)
      invert_permutation [T,k] int64     (:49-52)
      expert_offset    [E+1]   int64     (:54-60)
    """
    x = np.asarray(x, dtype=np.float32)
    T, H = x.shape
    if T == 0:
        raise ValueError("moe_select needs at least one token")
    if scores.shape != (T, num_experts):
        raise ValueError("scores shape mismatch")
    vals, idx = topk_desc(scores, k)                       # :40
    # softmax over the k kept logits (:41), fp32, one rounding to T1
    z = vals - vals[:, :1]
    e = np.exp(z.astype(np.float32)).astype(np.float32)
    w = e / e.sum(axis=1, keepdims=True, dtype=np.float32)
    expert_weights = round_to_dtype(w.astype(np.float32), dtype)
    flat = idx.reshape(-1)                                  # :42
    perm = np.argsort(flat, kind="stable")                  # :44 stable sort
    x_expand_permute = x[perm // k]                         # :45-47
    inv = np.empty(T * k, dtype=np.int64)                   # :49-52
    inv[perm] = np.arange(T * k, dtype=np.int64)
    counts = np.bincount(flat, minlength=num_experts)       # :54-60
    expert_offset = np.zeros(num_experts + 1, dtype=np.int64)
    expert_offset[1:] = np.cumsum(counts)
    return x_expand_permute, expert_weights, inv.reshape(T, k), expert_offset


def rows_with_ties(scores: np.ndarray, k: int) -> np.ndarray:
    """Boolean mask of rows whose top-(k+1) scores contain equal values, i.e.
    rows on which torch.topk's result is implementation defined."""
    s = np.asarray(scores, dtype=np.float32)
    kk = min(k + 1, s.shape[1])
    vals, _ = topk_desc(s, kk)
    return (np.diff(vals, axis=1) == 0).any(axis=1)


def detie_scores(scores: np.ndarray, dtype: str):
    """Make every row of `scores` free of duplicates by nudging duplicates down
    by one unit in the last place of `dtype` until unique.  Both the reference
    and the implementation under test then see identical, tie-free inputs.
    Returns (scores float32 exactly representable in dtype, number of nudges)."""
    s = round_to_dtype(scores, dtype).copy()
    nudges = 0

    def next_down(v: np.float32) -> np.float32:
        if dtype == "f32":
            return np.nextafter(np.float32(v), np.float32(-np.inf))
        if dtype == "f16":
            return np.float32(np.nextafter(np.float16(v), np.float16(-np.inf)))
        b = int(f32_to_bf16_bits(np.array([v], np.float32))[0])
        if v > 0:
            b -= 1
        elif v == 0:
            b = 0x8001
        else:
            b += 1
        return bf16_bits_to_f32(np.array([b], np.uint16))[0]

    for t in range(s.shape[0]):
        row = s[t]
        while True:
            srt = np.sort(row)
            if not (np.diff(srt) == 0).any():
                break
            seen = set()
            for e in range(row.shape[0]):
                v = float(row[e])
                while v in seen:
                    v = float(next_down(np.float32(v)))
                    nudges += 1
                seen.add(v)
                row[e] = v
    return s, nudges


# ----------------------------------------------------------------------------
# expert GEMMs, activation, combine
# ----------------------------------------------------------------------------
def moe_grouped_linear(x: np.ndarray, expert_offset: np.ndarray, w: np.ndarray,
                       bias: np.ndarray | None = None) -> np.ndarray:
    """torch_function/MoeColumnParallelLinear.py:58-69 and
    torch_function/MoeRowParallelLinear.py:44-55 (same loop): for every expert i
    rows [off[i], off[i+1]) of the output are X[rows] @ W[i].T (+ B[i]); all
    other rows stay zero (the zero-initialised output of :59 / :45).
    x [M,K], w [E,N,K], bias [E,N] | None -> [M,N] float32."""
    x = np.asarray(x, dtype=np.float32)
    M = x.shape[0]
    E, N, _ = w.shape
    y = np.zeros((M, N), dtype=np.float32)
    off = np.asarray(expert_offset).astype(np.int64)
    for i in range(E):
        r0, r1 = int(off[i]), int(off[i + 1])
        if r1 - r0 <= 0:
            continue
        acc = x[r0:r1].astype(np.float64) @ np.asarray(w[i], np.float32).astype(np.float64).T
        if bias is not None:
            acc = acc + np.asarray(bias[i], np.float64)
        y[r0:r1] = acc.astype(np.float32)
    return y


def swiglu(x: np.ndarray, beta: float = 1.0) -> np.ndarray:
    """torch_function/SwiGLU.py:15-16: first half is the gated (SiLU) input,
    second half the multiplier: Y = g * x * sigmoid(beta * x)."""
    x = np.asarray(x, dtype=np.float32)
    d = x.shape[-1] // 2
    a, g = x[..., :d].astype(np.float64), x[..., d:].astype(np.float64)
    return (g * a / (1.0 + np.exp(-beta * a))).astype(np.float32)


def silu_gate(x: np.ndarray, gate: np.ndarray | None = None) -> np.ndarray:
    """torch_function/SiLU.py:18-21: silu(X) (* gate)."""
    a = np.asarray(x, dtype=np.float64)
    y = a / (1.0 + np.exp(-a))
    if gate is not None:
        y = y * np.asarray(gate, dtype=np.float64)
    return y.astype(np.float32)


def skip_rms_norm(x: np.ndarray, weight: np.ndarray, skip: np.ndarray | None = None,
                  eps: float = 1e-5, dtype: str = "f32"):
    """torch_function/RMSNorm.py:42-56 (SkipRMSNorm.forward; RMSNorm.forward :15-24 when
    skip is None), over the last axis, with the reference's roundings to `dtype`:
    SkipOut = X + SkipIn (T1); Y = T1(float(SkipOut) * rsqrt(mean(SkipOut^2) + eps)) * weight (T1).
    Arrays are float32 holding exact up-casts.  Returns (Y, SkipOut)."""
    x = np.asarray(x, dtype=np.float32)
    s = x if skip is None else round_to_dtype(x + np.asarray(skip, np.float32), dtype)
    ms = np.mean(s.astype(np.float64) ** 2, axis=-1, keepdims=True)
    y1 = round_to_dtype((s.astype(np.float64) / np.sqrt(ms + eps)).astype(np.float32), dtype)
    y = round_to_dtype(y1 * np.asarray(weight, np.float32), dtype)
    return y, s


def moe_reduce(y: np.ndarray, expert_weights: np.ndarray,
               invert_permutation: np.ndarray, k: int) -> np.ndarray:
    """torch_function/MoeReduce.py:23-25: out[t] = sum_j w[t,j] * Y[inv[t,j]].
    y [T*k,N], expert_weights [T,k], invert_permutation [T,k] -> [T,N]."""
    y = np.asarray(y, dtype=np.float32)
    inv = np.asarray(invert_permutation).astype(np.int64).reshape(-1, k)
    w = np.asarray(expert_weights, dtype=np.float64).reshape(-1, k)
    g = y[inv].astype(np.float64)                      # [T,k,N]
    return (g * w[..., None]).sum(axis=1).astype(np.float32)


def moe_block(x, w_router, w_gate_up, w_down, num_experts, k, dtype="f32",
              scores=None, round_intermediates=True):
    """The Mixtral MoE feed-forward, model_zoo/mixtral/modeling/dynamic_batching/
    Model.py:187-214 with fused_ffn_glu=True: gate linear -> moe_select ->
    column-parallel [w1;w3] -> swiglu -> row-parallel w2 -> moe_reduce.

    All arrays float32 holding exact up-casts.  With round_intermediates the
    tensors that the operator API materialises in `dtype` (scores, x13, h,
    y) are rounded once to `dtype`, as the low-precision reference does between
    ops; without it the whole chain is the pure fp32 reference.
    Returns dict of every intermediate."""
    rd = (lambda a: round_to_dtype(a, dtype)) if round_intermediates else (lambda a: a)
    if scores is None:
        scores = rd((x.astype(np.float64) @ w_router.astype(np.float64).T).astype(np.float32))
    xe, ew, inv, off = moe_select(x, scores, num_experts, k, dtype)
    x13 = rd(moe_grouped_linear(xe, off, w_gate_up))
    h = rd(swiglu(x13))
    y = rd(moe_grouped_linear(h, off, w_down))
    out = moe_reduce(y, ew, inv, k)
    return dict(scores=scores, x_expand_permute=xe, expert_weights=ew,
                invert_permutation=inv, expert_offset=off, x13=x13, h=h, y=y, out=out)


# ----------------------------------------------------------------------------
# dense linear and decode-step cache attention (the operators around the MoE block)
# ----------------------------------------------------------------------------
def linear(x: np.ndarray, w: np.ndarray, b: np.ndarray | None = None) -> np.ndarray:
    """torch_function/Linear.py:32 (`F.linear(X, W, B)`), also the local product of
    ColumnParallelLinear.py:43 and RowParallelLinear.py:41 (+ bias at :44-45).
    x [*, K], w [N, K], b [N] | None -> [*, N] float32 (float64 accumulation)."""
    y = np.asarray(x, np.float64) @ np.asarray(w, np.float64).T
    if b is not None:
        y = y + np.asarray(b, np.float64)
    return y.astype(np.float32)


def cache_view(cache: np.ndarray, layout: int, layer_idx: int) -> np.ndarray:
    """View [rows, 2, heads, d] of one layer of a cache_mode-0 key/value cache in any of the
    four layouts (the index expressions of dynamic_batching/KeyValueCache.py:119-227)."""
    if layout == 0:      # [rows, layers, 2, heads, d]
        return cache[:, layer_idx]
    if layout == 1:      # [layers, rows, 2, heads, d]
        return cache[layer_idx]
    if layout == 2:      # [layers, 2, rows, heads, d]
        return cache[layer_idx].transpose(1, 0, 2, 3)
    if layout == 3:      # [layers, 2, heads, rows, d]
        return cache[layer_idx].transpose(2, 0, 1, 3)
    raise ValueError(f"unsupported cache_layout: {layout}")


def decode_cache_attention(q: np.ndarray, k_new: np.ndarray, v_new: np.ndarray, cache: np.ndarray,
                           cachestarts: np.ndarray, start_pos: np.ndarray, layout: int, layer_idx: int) -> np.ndarray:
    """One decode step of dynamic_batching.MultiHeadCacheAttention.forward
    (torch_function/dynamic_batching/MultiHeadCacheAttention.py:104-130) with one new token per
    sequence, cache_mode 0, no quantisation, no mask:
      KeyValueCache.forward (dynamic_batching/KeyValueCache.py:86-138): the new key / value of
      sequence b go to cache row cachestarts[b] + start_pos[b]; its keys / values are cache
      rows cachestarts[b] .. cachestarts[b] + start_pos[b];
      MultiHeadAttention.forward (dynamic_batching/MultiHeadAttention.py:56-108): kv heads are
      repeated for the query heads that share them, scores = q . K^T / sqrt(d), softmax, . V.
    q [B,Hq,d], k_new / v_new [B,Hkv,d]; `cache` (float32 values) is updated in place.
    -> [B,Hq,d] float32 (float64 accumulation, no intermediate rounding)."""
    B, Hq, d = q.shape
    Hkv = k_new.shape[1]
    rep = Hq // Hkv
    view = cache_view(cache, layout, layer_idx)            # [rows, 2, Hkv, d], a view: writes reach `cache`
    out = np.zeros((B, Hq, d), np.float32)
    for b in range(B):
        pos = int(start_pos[b])
        row = int(cachestarts[b]) + pos
        view[row, 0] = k_new[b]
        view[row, 1] = v_new[b]
        keys = view[int(cachestarts[b]):row + 1, 0].astype(np.float64)      # [kvlen, Hkv, d]
        vals = view[int(cachestarts[b]):row + 1, 1].astype(np.float64)
        for h in range(Hq):
            s = keys[:, h // rep] @ q[b, h].astype(np.float64) / np.sqrt(d)
            p = np.exp(s - s.max())
            p /= p.sum()
            out[b, h] = (p @ vals[:, h // rep]).astype(np.float32)
    return out
