"""B200-native implementation of the OPMX mixture-of-experts inference path.

    import ppl.pmx_b200.torch_function as OPMX      # moe_select, moe_*_parallel_linear, moe_reduce, swiglu, silu
    from ppl.pmx_b200.moe_layers import MoeFeedForward, patch_reference

The operators load the CUDA library on first use of `torch_function`; if it has
not been built (`python -m ppl.pmx_b200.build`) that import raises ImportError.
There is no CPU fallback.
"""
import importlib

__all__ = ["torch_function", "moe_layers", "workloads", "build"]


def __getattr__(name):
    if name in __all__:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
