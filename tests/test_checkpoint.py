"""Checkpoint shard format: the splitter and the MoE-layer loader of this package against
the reference's own SplitModel.split_pmx_model and Transformer.load_state_dict (staged,
unmodified, under oracle/_ref) on a toy Mixtral checkpoint.  CPU only: tensors are sliced
and copied, no kernel runs."""
import contextlib
import importlib
import io
import json
import os
import sys

import pytest
import torch

import oracle
from ppl.pmx_b200 import checkpoint as ck

PARAMS = dict(hidden_dim=64, intermediate_dim=96, num_layers=2, num_heads=8, num_kv_heads=4, vocab_size=48,
              num_experts=4, num_experts_per_token=2, norm_eps=1e-5)


def toy_state(seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    H, I, E, V = PARAMS["hidden_dim"], PARAMS["intermediate_dim"], PARAMS["num_experts"], PARAMS["vocab_size"]
    kv = H // PARAMS["num_heads"] * PARAMS["num_kv_heads"]
    st = {"tok_embeddings.weight": r(V, H), "norm.weight": r(H), "output.weight": r(V, H)}
    for n in range(PARAMS["num_layers"]):
        p = f"layers.{n}."
        st.update({p + "attention.wq.weight": r(H, H), p + "attention.wk.weight": r(kv, H),
                   p + "attention.wv.weight": r(kv, H), p + "attention.wo.weight": r(H, H),
                   p + "attention_norm.weight": r(H), p + "ffn_norm.weight": r(H),
                   p + "feed_forward.gate.weight": r(E, H), p + "feed_forward.w1.weight": r(E, I, H),
                   p + "feed_forward.w2.weight": r(E, H, I), p + "feed_forward.w3.weight": r(E, I, H)})
    return st


@pytest.mark.parametrize("shards", [1, 2, 4])
def test_split_matches_the_reference_splitter(tmp_path, shards):
    if oracle.ref_path() is None:
        pytest.skip("the OPMX reference is not staged (python oracle/make_ref.py)")
    src, ours, theirs = tmp_path / "merged", tmp_path / "ours", tmp_path / "theirs"
    src.mkdir()
    state = toy_state()
    torch.save(state, src / "model.pth")
    (src / "opmx_params.json").write_text(json.dumps(PARAMS))
    sys.path.insert(0, os.path.join(oracle.ref_path(), "model_zoo", "mixtral", "modeling"))
    try:
        ref_split = importlib.import_module("SplitModel")
    finally:
        sys.path.pop(0)
    ref_split.split_pmx_model(str(theirs), str(src), shards)
    ck.split_checkpoint(str(src), str(ours), shards)
    assert json.loads((ours / "opmx_params.json").read_text()) == json.loads((theirs / "opmx_params.json").read_text())
    for r in range(shards):
        a = ck.load_shard(str(ours), r, shards)
        b = torch.load(theirs / f"model.{r}.pth", map_location="cpu")
        assert sorted(a) == sorted(b)
        for key in a:
            assert torch.equal(a[key], b[key]), f"{key} differs in shard {r} of {shards}"
    with pytest.raises(ValueError):
        ck.load_shard(str(ours), 0, shards + 1)


def test_moe_layer_loads_like_the_reference_model():
    """w1 / w3 of a shard go into the fused wu exactly as Transformer.load_state_dict packs them
    (Model.py:399-413), for a 2-way tensor-parallel shard built without a process group."""
    if oracle.ref_path() is None:
        pytest.skip("the OPMX reference is not staged (python oracle/make_ref.py)")
    from ppl.pmx_b200.moe_layers import MoeFeedForward
    _, model_mod, ModelParams = oracle.import_reference_mixtral()
    state = toy_state(1)
    full = ck.split_state_dict(state, PARAMS, 1)[0]
    net = model_mod.Transformer(ModelParams(**PARAMS), False, True, True, True, False, False, False, 0, None)
    with contextlib.redirect_stdout(io.StringIO()):
        net.load_state_dict(full)
    for layer in range(PARAMS["num_layers"]):
        blk = MoeFeedForward(PARAMS["hidden_dim"], PARAMS["intermediate_dim"], PARAMS["num_experts"],
                             PARAMS["num_experts_per_token"], None, False)
        used = ck.load_moe_layer(blk, full, layer)
        assert len(used) == 4
        ref = net.layers[layer].feed_forward
        assert torch.equal(blk.gate.weight, ref.gate.weight)
        assert torch.equal(blk.wu.weight, ref.wu.weight)
        assert torch.equal(blk.w2.weight, ref.w2.weight)
    # a 2-way shard: this rank's wu is [w1 rows of its ffn slice ; w3 rows of the same slice]
    shards = ck.split_state_dict(state, PARAMS, 2)
    I = PARAMS["intermediate_dim"]
    for rank in range(2):
        # module shapes of a 2-way group without creating one: halve the ffn dimension
        blk = MoeFeedForward(PARAMS["hidden_dim"], I // 2, PARAMS["num_experts"], PARAMS["num_experts_per_token"], None, False)
        ck.load_moe_layer(blk, shards[rank], 0)
        lo, hi = rank * I // 2, (rank + 1) * I // 2
        assert torch.equal(blk.wu.weight[:, :I // 2], state["layers.0.feed_forward.w1.weight"][:, lo:hi])
        assert torch.equal(blk.wu.weight[:, I // 2:], state["layers.0.feed_forward.w3.weight"][:, lo:hi])
        assert torch.equal(blk.w2.weight, state["layers.0.feed_forward.w2.weight"][:, :, lo:hi])
    with pytest.raises(ValueError):
        ck.load_moe_layer(MoeFeedForward(32, I, 4, 2, None, False), full, 0)
    with pytest.raises(KeyError):
        ck.load_moe_layer(MoeFeedForward(PARAMS["hidden_dim"], I, 4, 2, None, False), {}, 0)
