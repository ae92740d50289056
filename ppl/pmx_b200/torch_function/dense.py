"""Dense linear operators of OPMX on the grouped expert-GEMM kernels.

`linear`, `column_parallel_linear` and `row_parallel_linear` keep the signatures, output
layouts and ONNX custom-op export of the reference operators
(torch_function/Linear.py:24-33, ColumnParallelLinear.py:28-57, RowParallelLinear.py:28-46).
The local product y = x . W^T (+ b) is the grouped kernel with ONE expert that owns all
rows (no offset table), so decode-size batches stream the weight rows once from HBM over
all SMs and prefill-size batches run on the paired-CTA tensor-core tiles.  The collectives
stay on the caller's process group: all-gather + concatenation along the last axis for
`gather_output`, all-reduce for the row-parallel sum.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .moe import _group_size, _require_cuda, moe_grouped_linear


def _local_linear(name: str, X: torch.Tensor, W: torch.Tensor, B: torch.Tensor | None) -> torch.Tensor:
    _require_cuda(name, X=X, W=W, B=B)
    if W.dim() != 2 or X.shape[-1] != W.shape[1]:
        raise ValueError(f"{name}: X has {X.shape[-1]} input features, W is {tuple(W.shape)}")
    if B is not None and tuple(B.shape) != (W.shape[0],):
        raise ValueError(f"{name}: B must be [{W.shape[0]}]")
    return moe_grouped_linear(X, None, W.unsqueeze(0), None if B is None else B.unsqueeze(0), zero_outside=False)


class Linear(torch.autograd.Function):
    """opmx::Linear (torch_function/Linear.py:6-33)."""

    @staticmethod
    def symbolic(g, X, W, B, in_features: int, out_features: int):
        if B is not None:
            return g.op("opmx::Linear", X, W, B, in_features_i=in_features, out_features_i=out_features,
                        bias_term_i=True)
        return g.op("opmx::Linear", X, W, in_features_i=in_features, out_features_i=out_features, bias_term_i=False)

    @staticmethod
    def forward(ctx, X, W, B, in_features: int, out_features: int):
        if torch.onnx.is_in_onnx_export():
            return torch.zeros(*X.shape[:-1], W.shape[0], dtype=W.dtype, device=X.device)
        return _local_linear("linear", X, W, B)


def linear(X: torch.Tensor, W: torch.Tensor, B: torch.Tensor | None, in_features: int, out_features: int):
    """Signature of torch_function/Linear.py:36-38.  Y = X W^T (+ B), fp32 accumulation,
    one rounding to X's dtype."""
    return Linear.apply(X, W, B, in_features, out_features)


def router_gate(X: torch.Tensor, W_router: torch.Tensor) -> torch.Tensor:
    """The router logits of the MoE block, scores = X . W_router^T (the `gate` call at
    model_zoo/mixtral/modeling/dynamic_batching/Model.py:188), for batches too large for
    the one-launch router + select kernel."""
    return _local_linear("router_gate", X, W_router, None)


class ColumnParallelLinear(torch.autograd.Function):
    """opmx::ColumnParallelLinear (torch_function/ColumnParallelLinear.py:7-57)."""

    @staticmethod
    def symbolic(g, X, W, B, proc_group, in_features: int, out_features: int, gather_output: bool = True):
        attrs = dict(in_features_i=in_features, out_features_i=out_features, gather_output_i=gather_output)
        if B is not None:
            return g.op("opmx::ColumnParallelLinear", X, W, B, bias_term_i=True, **attrs)
        return g.op("opmx::ColumnParallelLinear", X, W, bias_term_i=False, **attrs)

    @staticmethod
    def forward(ctx, X, W, B, proc_group, in_features: int, out_features: int, gather_output: bool = True):
        world = _group_size(proc_group)
        if torch.onnx.is_in_onnx_export():
            part = torch.zeros(*X.shape[:-1], W.shape[0], dtype=W.dtype, device=X.device)
            return torch.cat([part] * world, dim=-1) if gather_output and world > 1 else part
        y = _local_linear("column_parallel_linear", X, W, B)
        if gather_output and world > 1:
            parts = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(parts, y, group=proc_group)
            y = torch.cat(parts, dim=-1).contiguous()       # rank-major along the feature axis (:52)
        return y


def column_parallel_linear(X, W, B, proc_group, in_features: int, out_features: int,
                           gather_output: bool = True) -> torch.Tensor:
    """Signature of torch_function/ColumnParallelLinear.py:60-63.  W is this rank's
    [out_features/tp, in_features] shard."""
    return ColumnParallelLinear.apply(X, W, B, proc_group, in_features, out_features, gather_output)


class RowParallelLinear(torch.autograd.Function):
    """opmx::RowParallelLinear (torch_function/RowParallelLinear.py:7-46)."""

    @staticmethod
    def symbolic(g, X, W, B, proc_group, in_features: int, out_features: int, input_is_parallel: bool = False):
        attrs = dict(in_features_i=in_features, out_features_i=out_features, input_is_parallel_i=input_is_parallel)
        if B is not None:
            return g.op("opmx::RowParallelLinear", X, W, B, bias_term_i=True, **attrs)
        return g.op("opmx::RowParallelLinear", X, W, bias_term_i=False, **attrs)

    @staticmethod
    def forward(ctx, X, W, B, proc_group, in_features: int, out_features: int, input_is_parallel: bool = False):
        if not input_is_parallel:
            raise Exception("scatter input has not implement yet")      # as the reference (:34)
        if torch.onnx.is_in_onnx_export():
            return torch.zeros(*X.shape[:-1], W.shape[0], dtype=W.dtype, device=X.device)
        world = _group_size(proc_group)
        # the bias is added once, after the sum over ranks (:44-45); without a group it
        # goes into the GEMM epilogue
        y = _local_linear("row_parallel_linear", X, W, B if world == 1 else None)
        if world > 1:
            dist.all_reduce(y, group=proc_group)
            if B is not None:
                y = y + B
        return y


def row_parallel_linear(X, W, B, proc_group, in_features: int, out_features: int,
                        input_is_parallel: bool = False) -> torch.Tensor:
    """Signature of torch_function/RowParallelLinear.py:49-52.  W is this rank's
    [out_features, in_features/tp] shard; the partial products are all-reduced."""
    return RowParallelLinear.apply(X, W, B, proc_group, in_features, out_features, input_is_parallel)
