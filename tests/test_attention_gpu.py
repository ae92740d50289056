"""Decode-step attention over the key/value cache (pmx_decode_cache_attention behind
dynamic_batching.multi_head_cache_attention) against the golden vectors of the reference
operator and against the oracle on larger, ragged cases in every cache layout."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from tests.helpers import TORCH_DT, assert_close, dev, host, load
from tests.test_oracle_golden import ATTN, attention_fixture

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def DB():
    import ppl.pmx_b200.torch_function as F
    return F.dynamic_batching


@pytest.fixture(autouse=True, params=["mma", "simt"])
def attention_kernel(request, DB):
    """Every test runs once per attention kernel."""
    old = DB.set_decode_attention_kernel(request.param)
    yield request.param
    DB.set_decode_attention_kernel(old)


def run_op(DB, q, k, v, cache, cachestarts, start_pos, layout, layers, layer_idx, Hq, Hkv, D):
    B = q.shape[0]
    kvlens = start_pos + 1
    kvstarts = torch.cat([torch.zeros(1, dtype=torch.int64), torch.from_numpy(kvlens).cumsum(0)])
    return DB.multi_head_cache_attention(
        q, k, v, torch.arange(0, B + 1).cuda(), kvstarts.cuda(), torch.from_numpy(cachestarts).cuda(),
        torch.from_numpy(start_pos).cuda(), torch.tensor([B]), torch.tensor([1]), torch.tensor([int(kvlens.max())]),
        cache, None, None, Hq, D, True, False, Hkv, layers, layer_idx, 0, 8, 0, layout)


@pytest.mark.parametrize("name", ATTN)
def test_decode_attention_golden(DB, name):
    g, cache_in, cache_out = attention_fixture(name)
    dtype = str(g["dtype"])
    cache = dev(cache_in, dtype)
    out = run_op(DB, dev(g["q"], dtype), dev(g["k"], dtype), dev(g["v"], dtype), cache, g["cachestarts"],
                 g["start_pos"], int(g["layout"]), int(g["layers"]), int(g["layer_idx"]), int(g["num_heads"]),
                 int(g["num_kv_heads"]), int(g["head_dim"]))
    assert np.array_equal(host(cache), cache_out), "cache after the step differs from the reference's"
    assert_close(out, g["out"], dtype)


@pytest.mark.parametrize("layout", [0, 1, 2, 3])
@pytest.mark.parametrize("B,Hq,Hkv,D,maxpos,dtype", [(5, 8, 2, 128, 700, "f16"), (64, 4, 1, 128, 2048, "f16"),
                                                     (3, 8, 8, 64, 90, "bf16"), (1, 16, 2, 64, 0, "f16"),
                                                     (9, 32, 8, 128, 300, "bf16")])
def test_decode_attention_against_oracle(DB, layout, B, Hq, Hkv, D, maxpos, dtype):
    rng = np.random.default_rng(B * 31 + layout)
    layers, layer_idx = 3, 1
    start_pos = rng.integers(0, maxpos + 1, B).astype(np.int64)
    start_pos[0] = maxpos
    cap = maxpos + 3
    rows = B * cap
    shape = {0: (rows, layers, 2, Hkv, D), 1: (layers, rows, 2, Hkv, D), 2: (layers, 2, rows, Hkv, D),
             3: (layers, 2, Hkv, rows, D)}[layout]
    cache_np = orc.round_to_dtype(rng.standard_normal(shape).astype(np.float32), dtype)
    q = orc.round_to_dtype(rng.standard_normal((B, Hq, D)).astype(np.float32), dtype)
    k = orc.round_to_dtype(rng.standard_normal((B, Hkv, D)).astype(np.float32), dtype)
    v = orc.round_to_dtype(rng.standard_normal((B, Hkv, D)).astype(np.float32), dtype)
    cachestarts = (np.arange(B) * cap).astype(np.int64)
    rng.shuffle(cachestarts)                         # sequences need not be in cache order
    cache = dev(cache_np, dtype)
    out = run_op(DB, dev(q, dtype), dev(k, dtype), dev(v, dtype), cache, cachestarts, start_pos, layout, layers,
                 layer_idx, Hq, Hkv, D)
    want = orc.decode_cache_attention(q, k, v, cache_np, cachestarts, start_pos, layout, layer_idx)
    assert np.array_equal(host(cache), cache_np), "only the new rows of the layer may change, and to the new key / value"
    assert_close(out, want, dtype)


def test_decode_attention_refuses_what_it_does_not_cover(DB):
    B, Hq, Hkv, D = 2, 4, 2, 64
    q = torch.zeros(B, Hq, D, device="cuda", dtype=torch.float16)
    kv = torch.zeros(B, Hkv, D, device="cuda", dtype=torch.float16)
    cache = torch.zeros(40, 1, 2, Hkv, D, device="cuda", dtype=torch.float16)
    i64 = lambda *a: torch.tensor(a, dtype=torch.int64)
    args = dict(query=q, current_key=kv, current_value=kv, seqstarts=i64(0, 1, 2).cuda(), kvstarts=i64(0, 3, 6).cuda(),
                cachestarts=i64(0, 20).cuda(), start_pos=i64(2, 2).cuda(), decoding_batches=i64(B), max_seqlen=i64(1),
                max_kvlen=i64(3), cache=cache, scale=None, attn_mask=None, num_heads=Hq, head_dim=D, num_kv_heads=Hkv)
    DB.multi_head_cache_attention(**args)
    for change in (dict(max_seqlen=i64(4)), dict(cache_mode=1), dict(quant_bit=8), dict(is_alibi=True),
                   dict(decoding_batches=i64(1))):
        with pytest.raises(NotImplementedError):
            DB.multi_head_cache_attention(**{**args, **change})
    with pytest.raises(ValueError):
        DB.multi_head_cache_attention(**{**args, "cache_layout": 3})       # shape does not fit that layout
