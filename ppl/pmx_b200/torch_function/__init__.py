"""Drop-in replacements for the mixture-of-experts functions of
`pmx_llm.torch_function` (OPMX torch_function/__init__.py:17-20,37-38), the normalisation
in front of the block and the dense (column / row parallel) linears around it."""
from .moe import (moe_select, moe_column_parallel_linear, moe_row_parallel_linear, moe_reduce,
                  swiglu, silu, moe_grouped_linear, moe_dense_gate_up, moe_dense_mlp, moe_route_select, moe_norm_route_select, MoeSelect, MoeColumnParallelLinear,
                  MoeRowParallelLinear, MoeReduce, SwiGLU, SiLU, rms_norm, skip_rms_norm, RMSNorm, SkipRMSNorm)
from . import dynamic_batching
from .dense import (linear, router_gate, column_parallel_linear, row_parallel_linear, Linear, ColumnParallelLinear,
                    RowParallelLinear)

__all__ = ["moe_select", "moe_column_parallel_linear", "moe_row_parallel_linear", "moe_reduce",
           "swiglu", "silu", "moe_grouped_linear", "moe_route_select", "moe_norm_route_select", "rms_norm", "skip_rms_norm",
           "linear", "router_gate", "column_parallel_linear", "row_parallel_linear"]
