"""Checkpoint shards of the OPMX Mixtral model and their way into the MoE modules.

The reference splits a merged OPMX checkpoint into one `model.{rank}.pth` per tensor-parallel
rank (model_zoo/mixtral/modeling/SplitModel.py:23-92) and each rank loads its own file
(model_zoo/mixtral/modeling/Loader.py:52-59).  The sharding rules restated here:

  layers.N.attention.wq / wk / wv .weight   by heads: rows of whole heads, dim 0   (:41-48)
  layers.N.attention.wo.weight              input dimension, dim 1                 (:50)
  layers.N.feed_forward.w1 / w3 .weight     [E, I, H]: the ffn dimension, dim -2   (:51,53)
  layers.N.feed_forward.w2.weight           [E, H, I]: the ffn dimension, dim -1   (:52)
  tok_embeddings.weight                     embedding dimension, dim 1             (:65)
  output.weight                             vocabulary, dim 0                      (:66)
  biases of column-parallel linears         dim 0; wo / w2 biases and everything else
                                            (norms, router gate) are replicated    (:73-78)

A rank's fused projection is wu = [w1 shard ; w3 shard] along the output rows
(model_zoo/mixtral/modeling/dynamic_batching/Model.py:399-413), which is what
`load_moe_layer` writes into a `MoeFeedForward` (or any module with gate / wu / w2 members
of the reference's shapes).  Tensors are only sliced and copied; nothing is repacked.
"""
from __future__ import annotations

import json
import os
import re
from pathlib import Path
from typing import Mapping

import torch

_LAYER = re.compile(r"^layers\.(\d+)\.(attention|feed_forward)\.(\w+)\.(weight|bias)$")


def _split_even(t: torch.Tensor, shards: int, dim: int):
    if t.shape[dim] % shards:
        raise ValueError(f"dimension {dim} of size {t.shape[dim]} is not divisible by {shards} shards")
    return list(t.split(t.shape[dim] // shards, dim=dim))


def split_state_dict(state: Mapping[str, torch.Tensor], params: Mapping, num_shards: int) -> list[dict]:
    """Merged OPMX Mixtral state dict -> one state dict per tensor-parallel rank."""
    hidden = params["hidden_dim"]
    heads = params["num_heads"]
    kv_heads = params.get("num_kv_heads", heads) or heads
    head_dim = hidden // heads
    if heads % num_shards or kv_heads % num_shards:
        raise ValueError(f"{heads} query / {kv_heads} key-value heads are not divisible by {num_shards} shards")
    out = [dict() for _ in range(num_shards)]
    for key, value in state.items():
        m = _LAYER.match(key)
        parts = None
        if m and m.group(4) == "weight":
            where, leaf = m.group(2), m.group(3)
            if where == "attention" and leaf in ("wq", "wk", "wv"):
                n = heads if leaf == "wq" else kv_heads
                by_head = value.reshape(n, head_dim, hidden)
                parts = [p.reshape(-1, hidden) for p in _split_even(by_head, num_shards, 0)]
            elif where == "attention" and leaf == "wo":
                parts = _split_even(value, num_shards, 1)
            elif where == "feed_forward" and leaf in ("w1", "w3"):
                parts = _split_even(value, num_shards, -2)
            elif where == "feed_forward" and leaf == "w2":
                parts = _split_even(value, num_shards, -1)
        elif key == "tok_embeddings.weight":
            parts = _split_even(value, num_shards, 1)
        elif key == "output.weight":
            parts = _split_even(value, num_shards, 0)
        elif "bias" in key and "wo.bias" not in key and "w2.bias" not in key:
            parts = _split_even(value, num_shards, 0)
        for r in range(num_shards):
            out[r][key] = (parts[r] if parts is not None else value).clone()
    return out


def split_checkpoint(input_dir: str, output_dir: str, num_shards: int) -> None:
    """File-level form of split_state_dict: reads opmx_params.json and every *.pth of
    input_dir, writes opmx_params.json and model.{rank}.pth to output_dir."""
    os.makedirs(output_dir, exist_ok=True)
    with open(os.path.join(input_dir, "opmx_params.json")) as f:
        params = json.load(f)
    with open(os.path.join(output_dir, "opmx_params.json"), "w") as f:
        json.dump(params, f)
    state = {}
    for path in sorted(Path(input_dir).glob("*.pth")):
        state.update(torch.load(path, map_location="cpu"))
    for r, shard in enumerate(split_state_dict(state, params, num_shards)):
        torch.save(shard, os.path.join(output_dir, f"model.{r}.pth"))


def load_shard(ckpt_dir: str, rank: int, world_size: int) -> dict:
    """This rank's shard file, chosen as the reference loader does (sorted *.pth, one per rank)."""
    files = sorted(Path(ckpt_dir).glob("*.pth"))
    if len(files) != world_size:
        raise ValueError(f"Loading a checkpoint for MP={len(files)} but world size is {world_size}")
    return torch.load(files[rank], map_location="cpu")


@torch.no_grad()
def load_moe_layer(block, shard: Mapping[str, torch.Tensor], layer: int) -> list[str]:
    """Fills block.gate / block.wu / block.w2 (weights and, when present on both sides, biases)
    from a rank's shard.  Accepts the split form (w1, w3 -> packed into wu, gate rows first)
    and an already fused `wu`.  Returns the keys it consumed."""
    prefix = f"layers.{layer}.feed_forward."
    used = []

    def take(name):
        key = prefix + name
        if key in shard:
            used.append(key)
            return shard[key]
        return None

    def put(param, value, what):
        if tuple(param.shape) != tuple(value.shape):
            raise ValueError(f"{what}: checkpoint tensor {tuple(value.shape)} does not fit parameter {tuple(param.shape)}")
        param.copy_(value)

    gate = take("gate.weight")
    if gate is None:
        raise KeyError(prefix + "gate.weight")
    put(block.gate.weight, gate, "gate.weight")
    wu = take("wu.weight")
    local_ffn = block.wu.weight.shape[1] // 2
    if wu is not None:
        put(block.wu.weight, wu, "wu.weight")
    else:
        w1, w3 = take("w1.weight"), take("w3.weight")
        if w1 is None or w3 is None:
            raise KeyError(prefix + "w1.weight / w3.weight")
        put(block.wu.weight[:, :local_ffn, :], w1, "w1.weight")
        put(block.wu.weight[:, local_ffn:, :], w3, "w3.weight")
    w2 = take("w2.weight")
    if w2 is None:
        raise KeyError(prefix + "w2.weight")
    put(block.w2.weight, w2, "w2.weight")
    if getattr(block.wu, "bias", None) is not None:
        b1, b3 = take("w1.bias"), take("w3.bias")
        if b1 is not None and b3 is not None:
            put(block.wu.bias[:, :local_ffn], b1, "w1.bias")
            put(block.wu.bias[:, local_ffn:], b3, "w3.bias")
    if getattr(block.w2, "bias", None) is not None:
        b2 = take("w2.bias")
        if b2 is not None:
            put(block.w2.bias, b2, "w2.bias")
    return used
