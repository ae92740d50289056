"""Shared helpers of the parity tests."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
TAG = {v: k for k, v in TORCH_DT.items()}

# parity tolerance for fp16 / bf16 results against the fp32 reference
ATOL, RTOL = 2e-2, 1e-2
# fp32 tensors: exact fp32 multiply-add on both sides, only the order of the sums differs
ATOL32, RTOL32 = 2e-4, 1e-4


def load(name):
    return dict(np.load(os.path.join(GOLDEN, name), allow_pickle=False))


def dev(a, dtype, device="cuda"):
    """float32 numpy array (exactly representable in dtype) -> torch tensor on the GPU."""
    return torch.from_numpy(np.ascontiguousarray(a)).to(TORCH_DT[dtype]).to(device)


def host(t):
    return t.detach().float().cpu().numpy()


def tol(dtype):
    return dict(atol=ATOL32, rtol=RTOL32) if dtype == "f32" else dict(atol=ATOL, rtol=RTOL)


def assert_close(actual, expected, dtype, msg=""):
    np.testing.assert_allclose(host(actual) if isinstance(actual, torch.Tensor) else actual,
                               expected, err_msg=msg, **tol(dtype))


def assert_ulp(actual, expected, dtype, ulps=None, msg=""):
    eps = {"f32": 2.0 ** -23, "f16": 2.0 ** -10, "bf16": 2.0 ** -7}[dtype]
    if ulps is None:
        ulps = 4 if dtype == "f32" else 1
    a = host(actual) if isinstance(actual, torch.Tensor) else actual
    bad = np.abs(a - expected) > ulps * eps * np.maximum(np.abs(a), np.abs(expected)) + 1e-30
    assert not bad.any(), f"{msg}: {int(bad.sum())} elements differ by more than {ulps} ulp"
