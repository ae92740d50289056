"""CPU port of the OPMX MoE block, used ONLY to time the CPU baseline.

TEST / BENCHMARK INFRASTRUCTURE: the product package never imports this file.

It restates, with torch CPU tensors in the workload's dtype, the algorithm of
the reference operators as they run on host cores: top-k, softmax over the k
kept logits, stable sort, token gather (torch_function/MoeSelect.py:40-47),
one library GEMM per expert over its row range
(MoeColumnParallelLinear.py:61-67, MoeRowParallelLinear.py:47-53), SwiGLU
(SwiGLU.py:15-16), gather-multiply-sum combine (MoeReduce.py:23-25).  Two
interpreter loops of the reference (the T*k-iteration inverse permutation,
MoeSelect.py:49-52, and the offset scan, :54-60) are replaced by their
vectorised equivalents, which is faster than the reference; the baseline is
therefore, if anything, generous to the CPU.  Pinned against the golden
vectors of the reference in tests/test_oracle_golden.py.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def moe_select(x, scores, num_experts, k):
    T, H = x.shape
    w, idx = torch.topk(scores, k, dim=-1)                      # MoeSelect.py:40
    w = w.softmax(dim=-1)                                       # :41
    flat = idx.view(-1)
    sorted_ids, perm = flat.sort(stable=True)                   # :44
    xe = x.repeat_interleave(k, dim=0)[perm]                    # :45-47
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(T * k)                             # :49-52 vectorised
    counts = torch.bincount(flat, minlength=num_experts)        # :54-60 vectorised
    off = torch.zeros(num_experts + 1, dtype=torch.int64)
    off[1:] = counts.cumsum(0)
    return xe, w, inv.view(T, k), off


def grouped_linear(x, off, w, bias=None):
    E, N, _ = w.shape
    y = torch.zeros(x.shape[0], N, dtype=x.dtype)
    o = off.tolist()
    for i in range(E):                                          # MoeColumnParallelLinear.py:61-67
        if o[i + 1] - o[i] <= 0:
            continue
        y[o[i]:o[i + 1]] = F.linear(x[o[i]:o[i + 1]], w[i], bias[i] if bias is not None else None)
    return y


def swiglu(x, beta=1.0):
    a, g = torch.split(x, [x.shape[-1] // 2, x.shape[-1] // 2], -1)   # SwiGLU.py:15-16
    return g * a * torch.sigmoid(beta * a)


def moe_reduce(y, w, inv, k):
    out = y[inv].view(*w.shape, -1)                             # MoeReduce.py:24
    return (out * w.unsqueeze(-1)).sum(dim=-2)                  # :25


def moe_block(x, w_router, wu, w2, num_experts, k, scores=None):
    """model_zoo/mixtral/modeling/dynamic_batching/Model.py:187-214, fused_ffn_glu=True."""
    if scores is None:
        scores = F.linear(x, w_router)                          # Model.py:188
    xe, ew, inv, off = moe_select(x, scores, num_experts, k)
    h = swiglu(grouped_linear(xe, off, wu))
    y = grouped_linear(h, off, w2)
    return moe_reduce(y, ew, inv, k), (xe, ew, inv, off)
