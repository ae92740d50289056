"""The full-decoder harness of bench.py at toy width on one GPU: the reference's own Mixtral
Transformer (staged under oracle/_ref) runs one decode step with its own operators, with
patch_reference(), and with the fused MoE block swapped in; the logits must agree."""
import types

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_reference_decoder_step_with_the_operators_swapped_in():
    import oracle
    if oracle.ref_path() is None:
        pytest.skip("the OPMX reference is not staged (python oracle/make_ref.py)")
    import bench
    torch.cuda.set_device(0)
    ctx = bench.Ctx()
    ctx.world, ctx.rank, ctx.local_rank, ctx.group = 1, 0, 0, None
    ctx.device = torch.device("cuda", 0)
    ctx.peer_failed, ctx.blocks = False, {}
    ctx.args = types.SimpleNamespace(allreduce="auto", peer_algo="auto")
    cfg = dict(hidden_dim=512, intermediate_dim=1024, num_layers=3, num_heads=8, num_kv_heads=2, vocab_size=1024,
               num_experts=8, num_experts_per_token=2)
    out = bench.run_decoder(ctx, cfg, batch=12, cached=40, steps=2, parity_layers=2)
    for variant in ("patched", "fused", "fused+attention"):
        assert out["parity"][variant]["ok"], out["parity"]
        assert out["parity"][variant]["argmax_agree"] >= 0.9
    for variant in ("reference", "patched", "fused", "fused+attention"):
        assert out["timing"][variant]["ms_per_step"] > 0 and out["timing"][variant]["moe_ms_per_step"] > 0
