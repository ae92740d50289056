"""B200-native implementation of the OPMX mixture-of-experts inference path.

    import ppl.pmx_b200.torch_function as OPMX      # moe_select, moe_*_parallel_linear, moe_reduce, swiglu, silu
    from ppl.pmx_b200.moe_layers import MoeFeedForward, patch_reference
"""
from . import torch_function  # noqa: F401  (loads the CUDA library; fails loudly if it is missing)

__all__ = ["torch_function"]
