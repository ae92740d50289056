"""Seeded synthetic inputs with the shapes and value distributions of the MoE
layer workloads this package is measured on (Mixtral-8x7B decode / prefill, a
fine-grained 64-expert layer, and the small fp32 case).  Used by the benchmark,
the smoke test and the parity tests; there is no dataset or checkpoint behind
them: x ~ N(0,1), router weights ~ N(0,0.02), expert weights ~ N(0,1/sqrt(fan_in)).

Tensor-parallel layout follows the reference checkpoint splitter
(model_zoo/mixtral/modeling/SplitModel.py:54-56): w1, w3 [E,I,H] are split on I
(dim -2), w2 [E,H,I] on I (dim -1); the fused projection of a rank is
wu = [w1_shard ; w3_shard] (Model.py:399-413).
"""
from __future__ import annotations

from dataclasses import dataclass, replace

import numpy as np
import torch

TORCH_DTYPE = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


@dataclass(frozen=True)
class MoeShape:
    name: str
    T: int          # tokens
    H: int          # hidden size
    E: int          # experts
    k: int          # experts per token
    I: int          # intermediate (ffn) size per expert
    dtype: str      # "f16" | "bf16" | "f32"
    router_bias: str = "none"   # "zipf": per-expert additive logit bias (skewed load)
    force_empty: int = 0        # experts whose logits are forced to -1e4 (receive nothing)


def mixtral_decode(T: int) -> MoeShape:
    return MoeShape(f"mixtral_decode_t{T}", T, 4096, 8, 2, 14336, "f16")


WORKLOADS = {
    "small_f32": MoeShape("small_f32", 128, 1024, 8, 2, 3584, "f32"),
    **{f"decode_t{t}": mixtral_decode(t) for t in (1, 8, 32, 64, 128, 256)},
    "prefill": MoeShape("mixtral_prefill_t8192", 8192, 4096, 8, 2, 14336, "bf16"),
    "finegrained": MoeShape("finegrained_e64_k8", 4096, 2048, 64, 8, 1024, "f16", router_bias="zipf"),
    "finegrained_empty": MoeShape("finegrained_e64_k8_empty", 4096, 2048, 64, 8, 1024, "f16",
                                  router_bias="zipf", force_empty=8),
}


def scaled(shape: MoeShape, **kw) -> MoeShape:
    return replace(shape, **kw)


def _step_down(v: torch.Tensor) -> torch.Tensor:
    """Next representable value below v, in v's own dtype."""
    if v.dtype == torch.float32:
        return torch.nextafter(v, torch.full_like(v, -float("inf")))
    bits = v.view(torch.int16).to(torch.int32) & 0xFFFF
    pos = (bits & 0x8000) == 0
    zero = (bits & 0x7FFF) == 0
    nb = torch.where(pos, bits - 1, bits + 1)
    nb = torch.where(zero, torch.full_like(bits, 0x8001), nb)
    nb = torch.where(nb >= 0x8000, nb - 0x10000, nb)
    return nb.to(torch.int16).view(v.dtype)


def detie_(scores: torch.Tensor) -> int:
    """Remove equal values inside each row of `scores` [T,E] in place by moving
    duplicates down one unit in the last place at a time.  `torch.topk` orders
    equal scores in an implementation-defined way, so routing can only be
    compared bit for bit on rows without ties.  Returns the number of nudges."""
    nudges = 0
    for _ in range(64):
        srt, idx = torch.sort(scores.float(), dim=-1, descending=True, stable=True)
        dup = torch.zeros_like(srt, dtype=torch.bool)
        dup[:, 1:] = srt[:, 1:] == srt[:, :-1]
        n = int(dup.sum())
        if n == 0:
            return nudges
        nudges += n
        flat_dup = torch.zeros_like(dup)
        flat_dup.scatter_(1, idx, dup)
        scores[flat_dup] = _step_down(scores[flat_dup])
    raise RuntimeError("detie_: did not converge")


def zipf_bias(E: int) -> torch.Tensor:
    z = np.random.default_rng(0).zipf(1.2, E).astype(np.float64)
    return torch.from_numpy((3.0 * np.log(z) / np.log(z.max())).astype(np.float32))


def make_activations(shape: MoeShape, seed: int = 0, detie: bool = True):
    """x [T,H], router weight [E,H] and scores [T,E] on the CPU in shape.dtype."""
    dt = TORCH_DTYPE[shape.dtype]
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape.T, shape.H, generator=g).to(dt)
    w_router = (torch.randn(shape.E, shape.H, generator=g) * 0.02).to(dt)
    scores = (x.float() @ w_router.float().t())
    if shape.router_bias == "zipf":
        scores = scores + zipf_bias(shape.E)
    scores = scores.to(dt)
    if shape.force_empty:
        bias = zipf_bias(shape.E) if shape.router_bias == "zipf" else torch.arange(shape.E).float()
        lowest = torch.argsort(bias, stable=True)[: shape.force_empty]
        scores[:, lowest] = -1e4
    nudges = detie_(scores) if detie else 0
    return x, w_router, scores, nudges


def make_expert_weights(shape: MoeShape, device, seed: int = 0, tp_rank: int = 0, tp_size: int = 1):
    """This rank's wu [E, 2*I/tp, H] and w2 [E, H, I/tp] on `device`.  Each
    (tensor, expert) pair has its own generator seed, and the full I range is
    generated and then sliced, so shards of different ranks are slices of the
    same full tensors."""
    dt = TORCH_DTYPE[shape.dtype]
    E, H, I = shape.E, shape.H, shape.I
    assert I % tp_size == 0
    Il = I // tp_size
    lo, hi = tp_rank * Il, (tp_rank + 1) * Il
    dev = torch.device(device)
    wu = torch.empty(E, 2 * Il, H, dtype=dt, device=dev)
    w2 = torch.empty(E, H, Il, dtype=dt, device=dev)
    g = torch.Generator(device=dev)
    for e in range(E):
        for t, (dst, fan_in, full_shape) in enumerate((
                (wu[e, :Il], H, (I, H)), (wu[e, Il:], H, (I, H)), (w2[e], I, (H, I)))):
            g.manual_seed(seed * 1000003 + (t * 4096 + e) * 7 + 1)
            full = torch.randn(full_shape, generator=g, device=dev, dtype=torch.float32) / fan_in ** 0.5
            dst.copy_(full[lo:hi] if t < 2 else full[:, lo:hi])
            del full
    return wu, w2


def algorithmic_work(shape: MoeShape, tp_size: int = 1, active_experts: int | None = None):
    """FLOPs and minimum HBM bytes of one layer call on ONE rank with the
    operator API's materialised intermediates and SwiGLU fused into the gate/up
    GEMM: 6*T*k*H*I/tp flops; bytes = weights of the experts that own rows +
    activations each operator must read or write once."""
    b = {"f32": 4, "f16": 2, "bf16": 2}[shape.dtype]
    T, H, E, k = shape.T, shape.H, shape.E, shape.k
    Il = shape.I // tp_size
    act = E if active_experts is None else active_experts
    flops = 6.0 * T * k * H * Il
    w_gate_up = act * 2 * Il * H * b
    w_down = act * H * Il * b
    sel = T * H * b + T * E * b + T * k * H * b + T * k * b + T * k * 8 + (E + 1) * 8
    col = T * k * H * b + w_gate_up + T * k * Il * b
    row = T * k * Il * b + w_down + T * k * H * b
    red = T * k * H * b + T * k * (b + 8) + T * H * b
    return {"flops": flops, "bytes": float(sel + col + row + red),
            "bytes_select": float(sel), "bytes_gate_up": float(col), "bytes_down": float(row),
            "bytes_reduce": float(red), "flops_gate_up": 4.0 * T * k * H * Il,
            "flops_down": 2.0 * T * k * H * Il}
