"""pmx_moe_select_static: the moe_select entry point for hosts that cannot
allocate device memory around the call (its scratch is a fixed array inside the
library).  Called through the C ABI and compared with pmx_moe_select, which
takes a caller-provided workspace, on two calls in a row with different inputs
and shapes -- the second call finds the first call's leftovers in the scratch
and must not be affected by them.  Integer outputs and gathered rows must be
identical; the softmax weights come from the same kernel and must be identical
too.  Collected last so that a failure here cannot hide other tests.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(fn_static, x, sc, E, k):
    from ppl.pmx_b200._cabi import lib, check, ptr, stream_of, DTYPE_CODE
    T, H = x.shape
    outs = (torch.empty(T * k, H, dtype=x.dtype, device=x.device),
            torch.empty(T, k, dtype=x.dtype, device=x.device),
            torch.full((T, k), -7, dtype=torch.int64, device=x.device),
            torch.full((E + 1,), -7, dtype=torch.int64, device=x.device))
    code = DTYPE_CODE[x.dtype]
    if fn_static:
        check(lib.pmx_moe_select_static(ptr(x), ptr(sc), *(ptr(o) for o in outs), T, H, E, k, code, stream_of(x)))
    else:
        n = lib.pmx_moe_select_workspace_bytes(T, E, k)
        ws = torch.empty(n, dtype=torch.uint8, device=x.device)
        check(lib.pmx_moe_select(ptr(x), ptr(sc), *(ptr(o) for o in outs), T, H, E, k, code, ptr(ws), n, stream_of(x)))
    torch.cuda.synchronize()
    return outs


def test_static_scratch_select_matches_workspace_select_twice():
    from oracle import moe_oracle as orc
    torch.cuda.set_device(0)
    cases = [(5000, 64, 8, 2, torch.float16, 1), (2100, 40, 64, 8, torch.bfloat16, 2)]   # sizes that use the scratch
    for T, H, E, k, dt, seed in cases:
        # every case must take the three-launch path, the one that uses scratch (the
        # single-launch path covers up to 1024 tokens and 64 experts and needs none)
        assert T > 1024 or E > 64
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(T, H, generator=g).to(dt).cuda()
        sc = torch.randn(T, E, generator=g).to(dt).cuda()
        got = _call(True, x, sc, E, k)
        # the property the entry point exists for: with the outputs already allocated, a
        # call neither takes device memory from the driver nor from torch's allocator
        torch.cuda.synchronize()
        free0, _ = torch.cuda.mem_get_info()
        torch_allocs0 = torch.cuda.memory_stats()["allocation.all.allocated"]
        from ppl.pmx_b200._cabi import lib, check, ptr, stream_of, DTYPE_CODE
        check(lib.pmx_moe_select_static(ptr(x), ptr(sc), *(ptr(o) for o in got), T, H, E, k, DTYPE_CODE[dt], stream_of(x)))
        torch.cuda.synchronize()
        assert torch.cuda.memory_stats()["allocation.all.allocated"] == torch_allocs0
        assert torch.cuda.mem_get_info()[0] == free0, "device memory changed around pmx_moe_select_static"
        want = _call(False, x, sc, E, k)
        for a, b, name in zip(got, want, ("x_expand_permute", "expert_weights", "invert_permutation", "expert_offset")):
            assert torch.equal(a, b), f"{name} differs between the two entry points (T={T}, E={E}, k={k})"
        # and both agree with the oracle's routing on tie-free rows
        s32 = sc.float().cpu().numpy()
        if not orc.rows_with_ties(s32, k).any():
            _, _, inv, off = orc.moe_select(x.float().cpu().numpy(), s32, E, k)
            assert np.array_equal(got[3].cpu().numpy(), off) and np.array_equal(got[2].cpu().numpy(), inv)


def test_static_scratch_select_rejects_oversized_problems():
    from ppl.pmx_b200._cabi import lib, PmxError
    torch.cuda.set_device(0)
    T, H, E, k = 400000, 8, 8, 2          # ids alone need 3.2 MB > the 1 MiB scratch
    assert lib.pmx_moe_select_workspace_bytes(T, E, k) > (1 << 20)
    x = torch.zeros(T, H, dtype=torch.float16, device="cuda")
    sc = torch.zeros(T, E, dtype=torch.float16, device="cuda")
    with pytest.raises(PmxError) as err:
        _call(True, x, sc, E, k)
    assert err.value.status == -4 and "built-in scratch" in str(err.value)
