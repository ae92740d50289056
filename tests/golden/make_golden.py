"""Generate the golden fixtures under tests/golden/ by running the OPMX
reference operators themselves on CPU.

Usage (only where the OPMX tree is available; it is not needed to RUN the
tests, the produced .npz/.json files are committed):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference <path to OPMX tree>

Every low-precision tensor is stored as its exact float32 up-cast together
with a `dtype` tag, so that the fixtures need nothing but numpy to load.
The torch version used is recorded in each file.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import moe_oracle as orc  # noqa: E402  (de-tie helper only)

TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def gen_inputs(seed, T, H, E, dtype, lead=None, bias=None, force_empty=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g)
    wr = torch.randn(E, H, generator=g) * 0.02
    dt = TORCH_DT[dtype]
    x = x.to(dt)
    scores = torch.nn.functional.linear(x.float(), wr).to(dt).float()
    if bias is not None:
        scores = (scores + torch.from_numpy(bias).float()).to(dt).float()
    if force_empty:
        scores[:, :force_empty] = -1e4
        scores = scores.to(dt).float()
    s_np, nudges = orc.detie_scores(scores.numpy(), dtype)
    scores = torch.from_numpy(s_np).to(dt)
    assert np.array_equal(scores.float().numpy(), s_np)
    if lead is not None:
        x = x.view(*lead, H)
        scores = scores.view(*lead, E)
    return x, scores, nudges


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import torch_function as OPMX  # the reference operators

    meta = {"torch": torch.__version__}

    # ---------------------------------------------------------------- select
    select_cases = [
        # name, seed, T, H, E, k, dtype, lead, zipf-bias, force_empty
        ("select_f32_mixtral", 0, 37, 24, 8, 2, "f32", None, False, 0),
        ("select_f16_mixtral", 1, 64, 32, 8, 2, "f16", None, False, 0),
        ("select_bf16_mixtral", 2, 200, 16, 8, 2, "bf16", None, False, 0),
        ("select_f16_fine_empty", 3, 96, 16, 64, 8, "f16", None, True, 8),
        ("select_f16_single_token", 4, 1, 40, 8, 2, "f16", None, False, 0),
        ("select_f32_k_equals_e", 5, 9, 8, 4, 4, "f32", None, False, 0),
        ("select_bf16_leading_dims", 6, 10, 64, 8, 2, "bf16", (2, 5), False, 0),
        ("select_f16_one_expert", 7, 33, 8, 8, 1, "f16", None, False, 7),
        ("select_f32_odd_experts", 8, 50, 12, 5, 3, "f32", None, False, 0),
        ("select_f16_many_tokens", 9, 1500, 8, 8, 2, "f16", None, False, 0),
    ]
    for name, seed, T, H, E, k, dtype, lead, zipf, empty in select_cases:
        bias = None
        if zipf:
            z = np.random.default_rng(0).zipf(1.2, E).astype(np.float64)
            bias = (3.0 * np.log(z) / np.log(z.max())).astype(np.float32)
        x, scores, nudges = gen_inputs(seed, T, H, E, dtype, lead, bias, empty)
        torch.set_default_dtype(TORCH_DT[dtype])
        xe, ew, inv, off = OPMX.moe_select(x, scores, E, k)
        torch.set_default_dtype(torch.float32)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"), dtype=dtype, E=E, k=k, nudges=nudges,
            x=f32(x), scores=f32(scores), x_expand_permute=f32(xe),
            expert_weights=f32(ew), invert_permutation=inv.numpy().astype(np.int64),
            expert_offset=off.numpy().astype(np.int64), **meta)
        print(name, "offsets", off.tolist()[:9], "nudges", nudges)

    # ------------------------------------------------------- linears / swiglu
    g = torch.Generator().manual_seed(20)
    E, K, N, M = 8, 40, 48, 80
    for dtype in ("f32", "f16", "bf16"):
        dt = TORCH_DT[dtype]
        x = torch.randn(10, E, K, generator=g).to(dt)
        w = (torch.randn(E, N, K, generator=g) / K ** 0.5).to(dt)
        b = torch.randn(E, N, generator=g).to(dt)
        # the reference's own __main__ offsets: arange(E+1) over 80 rows, so
        # rows 8.. stay zero (MoeColumnParallelLinear.py:135-136)
        off_a = torch.arange(E + 1)
        # ragged with empty experts, not covering the first/last rows
        off_b = torch.tensor([3, 3, 20, 20, 21, 50, 50, 64, 77])
        torch.set_default_dtype(dt)
        out = {}
        for tag, off in (("arange", off_a), ("ragged", off_b)):
            out["col_bias_" + tag] = f32(OPMX.moe_column_parallel_linear(x, off, w, b, None, E, K, N, False))
            out["col_nobias_" + tag] = f32(OPMX.moe_column_parallel_linear(x, off, w, None, None, E, K, N, False))
            out["row_nobias_" + tag] = f32(OPMX.moe_row_parallel_linear(x, off, w, None, None, E, K, N, True))
        x13 = torch.randn(7, 3, 2 * 36, generator=g).to(dt)
        out["swiglu_in"] = f32(x13)
        out["swiglu_out"] = f32(OPMX.swiglu(x13))
        out["swiglu_out_beta"] = f32(OPMX.swiglu(x13, 1.7))
        a, c = x13[..., :36].contiguous(), x13[..., 36:].contiguous()
        out["silu_gate_out"] = f32(OPMX.silu(a, c))
        out["silu_out"] = f32(OPMX.silu(a))
        torch.set_default_dtype(torch.float32)
        np.savez_compressed(
            os.path.join(HERE, f"linear_{dtype}.npz"), dtype=dtype, x=f32(x), w=f32(w), b=f32(b),
            off_arange=off_a.numpy(), off_ragged=off_b.numpy(), **out, **meta)
        print("linear", dtype)

    # ------------------------------------------------------------- reduce
    g = torch.Generator().manual_seed(30)
    for dtype in ("f32", "f16", "bf16"):
        dt = TORCH_DT[dtype]
        T, k, N = 21, 4, 56
        y = torch.randn(T, k, N, generator=g).to(dt)
        w = torch.rand(T, k, generator=g).to(dt)
        inv = torch.randperm(T * k, generator=g).view(T, k)
        out = OPMX.moe_reduce(y, w, inv, k)
        np.savez_compressed(
            os.path.join(HERE, f"reduce_{dtype}.npz"), dtype=dtype, k=k, y=f32(y),
            expert_weights=f32(w), invert_permutation=inv.numpy(), out=f32(out), **meta)
        print("reduce", dtype)

    # ------------------------------------------------------------ rms norm
    g = torch.Generator().manual_seed(35)
    for dtype in ("f32", "f16", "bf16"):
        dt = TORCH_DT[dtype]
        x = torch.randn(3, 11, 96, generator=g).to(dt)
        sk = torch.randn(3, 11, 96, generator=g).to(dt)
        w = (1 + 0.1 * torch.randn(96, generator=g)).to(dt)
        y_skip, s_out = OPMX.skip_rms_norm(x, w, sk, -1, 1e-5)
        y_noskip, s_same = OPMX.skip_rms_norm(x, w, None, -1, 1e-6)
        y_plain = OPMX.rms_norm(x, w, -1, 1e-5)
        assert torch.equal(s_same, x)
        np.savez_compressed(os.path.join(HERE, f"rmsnorm_{dtype}.npz"), dtype=dtype, x=f32(x), skip=f32(sk),
                            weight=f32(w), y_skip=f32(y_skip), skip_out=f32(s_out), y_noskip=f32(y_noskip),
                            y_plain=f32(y_plain), **meta)
        print("rmsnorm", dtype)

    # ------------------------------------------- whole block (Model.py:187-214)
    def block(x, wr, wu, wd, E, k, dt):
        torch.set_default_dtype(dt)
        H, I = x.shape[-1], wd.shape[-1]
        scores = OPMX.linear(x, wr, None, H, E)
        xe, ew, inv, off = OPMX.moe_select(x, scores, E, k)
        x13 = OPMX.moe_column_parallel_linear(xe, off, wu, None, None, E, H, 2 * I, False)
        h = OPMX.swiglu(x13)
        y = OPMX.moe_row_parallel_linear(h, off, wd, None, None, E, I, H, True)
        out = OPMX.moe_reduce(y, ew, inv, k)
        torch.set_default_dtype(torch.float32)
        return scores, xe, ew, inv, off, x13, h, y, out

    for name, seed, T, H, E, k, I, dtype in [
        ("block_f32", 40, 48, 64, 8, 2, 96, "f32"),
        ("block_f16", 41, 48, 64, 8, 2, 96, "f16"),
        ("block_bf16", 42, 70, 128, 8, 2, 160, "bf16"),
        ("block_f16_fine", 43, 64, 64, 16, 4, 32, "f16"),
    ]:
        g = torch.Generator().manual_seed(seed)
        dt = TORCH_DT[dtype]
        x = torch.randn(T, H, generator=g).to(dt)
        wr = (torch.randn(E, H, generator=g) * 0.02).to(dt)
        w1 = (torch.randn(E, I, H, generator=g) / H ** 0.5).to(dt)
        w3 = (torch.randn(E, I, H, generator=g) / H ** 0.5).to(dt)
        wd = (torch.randn(E, H, I, generator=g) / I ** 0.5).to(dt)
        wu = torch.cat([w1, w3], dim=1).contiguous()
        # low-precision run of the reference
        lo = block(x, wr, wu, wd, E, k, dt)
        # fp32 run of the reference with the routing of the low-precision scores
        torch.set_default_dtype(torch.float32)
        sc = lo[0]
        xe, ew, inv, off = OPMX.moe_select(x.float(), sc.float(), E, k)
        x13 = OPMX.moe_column_parallel_linear(xe, off, wu.float(), None, None, E, H, 2 * I, False)
        h = OPMX.swiglu(x13)
        y = OPMX.moe_row_parallel_linear(h, off, wd.float(), None, None, E, I, H, True)
        out32 = OPMX.moe_reduce(y, ew, inv, k)
        ties = int(orc.rows_with_ties(f32(sc), k).sum())
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"), dtype=dtype, E=E, k=k, tied_rows=ties,
            x=f32(x), w_router=f32(wr), w_gate_up=f32(wu), w_down=f32(wd),
            scores=f32(lo[0]), x_expand_permute=f32(lo[1]), expert_weights=f32(lo[2]),
            invert_permutation=lo[3].numpy(), expert_offset=lo[4].numpy(),
            x13=f32(lo[5]), h=f32(lo[6]), y=f32(lo[7]), out=f32(lo[8]),
            out_fp32_reference=f32(out32), **meta)
        print(name, "tied rows", ties, "offsets", lo[4].tolist())

    # ------------------------------------------------ ONNX graph of the block
    from torch.onnx._internal.torchscript_exporter import utils as U, _globals

    class M(torch.nn.Module):
        def __init__(s):
            super().__init__()
            s.wu = torch.nn.Parameter(torch.randn(8, 64, 32))
            s.wd = torch.nn.Parameter(torch.randn(8, 32, 32))
            s.bu = torch.nn.Parameter(torch.randn(8, 64))

        def forward(s, X, S):
            xe, ew, inv, off = OPMX.moe_select(X, S, 8, 2)
            h = OPMX.swiglu(OPMX.moe_column_parallel_linear(xe, off, s.wu, s.bu, None, 8, 32, 64, False))
            y = OPMX.moe_row_parallel_linear(h, off, s.wd, None, None, 8, 32, 32, True)
            return OPMX.moe_reduce(y, ew, inv, 2)

    _globals.GLOBALS.export_onnx_opset_version = 11
    _globals.GLOBALS.in_onnx_export = True
    m = M()
    with U.exporter_context(m, torch.onnx.TrainingMode.EVAL, False):
        graph, _, _ = U._model_to_graph(m, (torch.randn(4, 32), torch.randn(4, 8)), do_constant_folding=False)
    _globals.GLOBALS.in_onnx_export = False
    nodes = []
    for n in graph.nodes():
        if not n.kind().startswith("opmx::"):
            continue
        attrs = {a: (n.f(a) if n.kindOf(a) == "f" else n.i(a)) for a in n.attributeNames()}
        nodes.append({"kind": n.kind(), "attrs": attrs,
                      "n_inputs": len(list(n.inputs())), "n_outputs": len(list(n.outputs()))})
    with open(os.path.join(HERE, "onnx_block_graph.json"), "w") as f:
        json.dump({"torch": torch.__version__, "nodes": nodes}, f, indent=1)
    print("onnx nodes", [n["kind"] for n in nodes])


if __name__ == "__main__":
    main()
