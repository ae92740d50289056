"""CPU checkers for the CUDA path.  TEST / BENCHMARK INFRASTRUCTURE ONLY: nothing under
this directory is imported by the product package.

moe_oracle.py  numpy restatement of the OPMX MoE operators (the parity oracle)
cpu_port.py    torch-CPU restatement used to time a CPU baseline when the staged
               reference is absent
make_ref.py    stages the unmodified OPMX reference (pure Python) under oracle/_ref/
"""
from __future__ import annotations

import importlib
import os
import sys

_REF = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def ref_path() -> str | None:
    """Directory holding the staged OPMX reference, or None if it has not been staged."""
    return _REF if os.path.isdir(os.path.join(_REF, "torch_function")) else None


def import_reference():
    """-> the reference's `torch_function` module (its operators run on CPU or CUDA torch
    tensors), imported from oracle/_ref/.  Raises ImportError when it is not staged."""
    path = ref_path()
    if path is None:
        raise ImportError("the OPMX reference is not staged: run `python oracle/make_ref.py --src <OPMX tree>`")
    if path not in sys.path:
        sys.path.insert(0, path)
    return importlib.import_module("torch_function")


def import_reference_mixtral():
    """-> (torch_function module, Mixtral dynamic-batching Model module, ModelParams class)."""
    opmx = import_reference()
    zoo = os.path.join(ref_path(), "model_zoo")
    for p in (zoo, os.path.join(zoo, "mixtral", "modeling", "dynamic_batching")):
        if p not in sys.path:
            sys.path.insert(0, p)
    model = importlib.import_module("Model")
    params = importlib.import_module("ModelParams").ModelParams
    return opmx, model, params
