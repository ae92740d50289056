"""The measured workloads at their full BASELINE sizes.  The oracle's integer routing is
cheap at any size, so routing is compared bit for bit; the floating-point stages are
checked through size-independent properties and on sampled rows against fp32 math.
"""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from tests.helpers import ATOL, RTOL, host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def F():
    import ppl.pmx_b200.torch_function as F
    return F


@pytest.mark.parametrize("wl", ["decode_t256", "prefill", "finegrained", "finegrained_empty"])
def test_full_size_routing_is_bit_exact_and_round_trips(F, wl):
    from ppl.pmx_b200 import workloads as W
    sh = W.WORKLOADS[wl]
    x, _, sc, _ = W.make_activations(sh)
    xd, sd = x.cuda(), sc.cuda()
    xe, ew, inv, off = F.moe_select(xd, sd, sh.E, sh.k)
    s32 = sc.float().numpy()
    assert not orc.rows_with_ties(s32, sh.k).any()
    _, oew, oinv, ooff = orc.moe_select(np.zeros((sh.T, 1), np.float32), s32, sh.E, sh.k, sh.dtype)
    assert np.array_equal(off.cpu().numpy(), ooff)
    assert np.array_equal(inv.cpu().numpy(), oinv)
    if wl == "finegrained_empty":
        assert int((np.diff(ooff) == 0).sum()) == 8
    # every slot's row is a bit-exact copy of its token
    flat = xe.view(-1, sh.H)
    assert torch.equal(flat[inv.view(-1)], xd.repeat_interleave(sh.k, dim=0))
    # expert_weights: one rounding of the fp32 softmax (within 1 ulp)
    eps = {"f16": 2.0 ** -10, "bf16": 2.0 ** -7}[sh.dtype]
    assert np.all(np.abs(host(ew) - oew) <= eps * np.maximum(host(ew), oew) + 1e-30)
    # dispatch -> combine round trip: the weights of a token sum to 1, so combining the
    # gathered rows gives the token back
    back = F.moe_reduce(xe, ew, inv, sh.k)
    np.testing.assert_allclose(host(back), host(xd), atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("wl", ["decode_t64", "prefill", "finegrained", "finegrained_empty"])
def test_full_size_expert_gemms_on_sampled_rows(F, wl):
    """Both grouped GEMMs of the Mixtral layer at full size: sampled rows of every expert
    against fp32 matmuls on the same device, and linearity of the down projection."""
    from ppl.pmx_b200 import workloads as W
    from ppl.pmx_b200.torch_function.moe import moe_grouped_linear
    sh = W.WORKLOADS[wl]
    x, _, sc, _ = W.make_activations(sh)
    wu, w2 = W.make_expert_weights(sh, "cuda")
    xe, ew, inv, off = F.moe_select(x.cuda(), sc.cuda(), sh.E, sh.k)
    flat = xe.view(-1, sh.H)
    h = moe_grouped_linear(flat, off, wu, None, swiglu=True, zero_outside=False)
    y = moe_grouped_linear(h, off, w2, None, zero_outside=False)
    torch.cuda.synchronize()
    offs = off.cpu().tolist()
    rng = np.random.default_rng(0)
    I = sh.I
    for e in range(sh.E):
        r0, r1 = offs[e], offs[e + 1]
        if r1 <= r0:
            continue
        rows = torch.from_numpy(rng.choice(np.arange(r0, r1), size=min(8, r1 - r0), replace=False)).cuda()
        xr = flat[rows].float()
        gu = xr @ wu[e].float().t()
        gate, up = gu[:, :I], gu[:, I:]
        h_ref = up * gate * torch.sigmoid(gate)
        torch.testing.assert_close(h[rows].float(), h_ref, atol=ATOL, rtol=RTOL)
        y_ref = h[rows].float() @ w2[e].float().t()
        torch.testing.assert_close(y[rows].float(), y_ref, atol=ATOL, rtol=RTOL)
    # linearity of the down projection: doubling the input doubles every fp32 partial sum
    # exactly, so f(2h) = 2 f(h) bit for bit wherever the result is a normal number
    y2 = moe_grouped_linear(h * 2, off, w2, None, zero_outside=False)
    normal = y.abs() > 1e-3
    assert torch.equal(y2[normal], (y * 2)[normal])
    torch.testing.assert_close(y2.float(), y.float() * 2, atol=1e-6, rtol=1e-3)
    # and the whole layer against the per-row fp32 chain on a few tokens
    out = F.moe_reduce(y.view(sh.T, sh.k, -1), ew, inv, sh.k)
    for t in rng.choice(sh.T, size=4, replace=False):
        acc = torch.zeros(sh.H, device="cuda")
        for j in range(sh.k):
            acc += ew[t, j].float() * y[inv[t, j]].float()
        torch.testing.assert_close(out[t].float(), acc, atol=ATOL, rtol=RTOL)
