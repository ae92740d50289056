"""CPU-only checks of the host side: the C-ABI library loads and exports every
symbol the header declares, argument errors come back as status codes before
any launch, operators refuse CPU tensors, ONNX export emits the reference's
custom-op graph, and the workload / module helpers have the reference's shapes."""
import ctypes as C
import json
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from ppl.pmx_b200.build import build
    build()
    from ppl.pmx_b200 import _cabi
    return _cabi.lib


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "pmx_moe.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    names = sorted(set(re.findall(r"\b(pmx_[a-z0-9_]+)\s*\(", header)))
    assert len(names) >= 13
    raw = C.CDLL(os.path.join(ROOT, "ppl", "pmx_b200", "libpmx_moe_b200.so"))
    for n in names:
        assert hasattr(raw, n), f"{n} declared in pmx_moe.h but not exported"
    assert lib.pmx_moe_abi_version() == 3
    assert lib.pmx_moe_status_string(-4) == b"workspace missing or too small"


def test_workspace_sizes_and_argument_errors_without_a_gpu(lib):
    from ppl.pmx_b200._cabi import GemmPlan
    assert lib.pmx_moe_select_workspace_bytes(0, 8, 2) == 0
    n = lib.pmx_moe_select_workspace_bytes(8192, 8, 2)
    assert n >= 8192 * 2 * 4 and n % 16 == 0
    # Mixtral down projection: 64 tokens -> enough work for every SM, status words only;
    # one token (2 rows) -> K is sliced: fp32 partial sums + status words
    assert lib.pmx_moe_grouped_linear_workspace_bytes(128, 4096, 14336, 8, 0, 0, None) == 256
    for plan in (None, C.byref(GemmPlan(balance=2))):
        ws = lib.pmx_moe_grouped_linear_workspace_bytes(2, 4096, 14336, 8, 0, 0, plan)
        assert ws > 256 and (ws - 256) % (2 * 4096 * 4) == 0
    assert lib.pmx_moe_grouped_linear_workspace_bytes(128, 4096, 14336, 8, 2, 0, None) == 256   # fp32 -> CUDA cores
    assert lib.pmx_moe_grouped_linear_workspace_bytes(128, 4097, 64, 8, 0, 1, None) == 0        # odd N with SwiGLU
    assert b"even N" in lib.pmx_moe_last_error()
    bad = GemmPlan(kernel=1, tile_feat=24)
    assert lib.pmx_moe_grouped_linear_workspace_bytes(1024, 256, 128, 8, 0, 0, C.byref(bad)) == 0
    # argument checks return before anything is launched
    one = C.c_void_p(16)
    assert lib.pmx_moe_select(one, one, one, one, one, one, 4, 8, 8, 9, 0, one, 1 << 20, None) == -1
    assert b"exceeds the number of experts" in lib.pmx_moe_last_error()
    assert lib.pmx_moe_select(one, one, one, one, one, one, 0, 8, 8, 2, 0, one, 1 << 20, None) == -1
    assert lib.pmx_moe_select(one, one, one, one, one, one, 4, 8, 8, 2, 0, one, 8, None) == -4
    assert lib.pmx_moe_select(None, one, one, one, one, one, 4, 8, 8, 2, 0, one, 1 << 20, None) == -1
    assert lib.pmx_moe_select(one, one, one, one, one, one, 4, 8, 8, 2, 7, one, 1 << 20, None) == -2
    assert lib.pmx_moe_reduce(one, one, one, one, 0, 2, 8, 0, None) == -1
    assert lib.pmx_swiglu(one, one, 4, 7, 1.0, 0, None) == -1
    assert lib.pmx_moe_grouped_linear(one, one, one, None, one, 4, 8, 0, 2, 0, 0, 1.0, 1, None, one, 256, None) == -1
    assert lib.pmx_moe_select_static(one, one, one, one, one, one, 10 ** 7, 8, 8, 2, 0, None) == -4
    # fused front ends: decode-size batches only, otherwise "use the stand-alone operators"
    assert lib.pmx_moe_route_select_workspace_bytes(64, 4096, 8, 2, 0) == 64 + 64 * 8
    assert lib.pmx_moe_route_select_workspace_bytes(2000, 4096, 8, 2, 0) == 0        # too many tokens
    assert lib.pmx_moe_route_select_workspace_bytes(64, 4096, 65, 2, 0) == 0         # too many experts
    assert lib.pmx_moe_route_select_workspace_bytes(64, 4100, 8, 2, 0) == 0          # rows not 16-byte multiples
    assert lib.pmx_moe_norm_route_select_workspace_bytes(64, 4096, 8, 2, 0) == 64 + 64 * 8
    assert lib.pmx_moe_norm_route_select_workspace_bytes(1024, 16384, 8, 2, 0) == 0  # rows do not fit on chip
    assert lib.pmx_moe_route_select(one, one, one, one, one, one, one, 5000, 64, 8, 2, 0, one, 1 << 20, None) == -2
    assert lib.pmx_moe_norm_route_select(one, None, None, 1e-5, one, None, one, one, one, one, one, 8, 64, 8, 2, 0,
                                         one, 1 << 20, None) == -1                    # norm weight missing
    assert lib.pmx_skip_rms_norm(one, one, one, one, None, 4, 64, 1e-5, 0, None) == -1  # skip without skip_out
    # exchange buffer: 16 KB of control + two areas of one 32-byte slot per 16-byte item (+ 8 warps of slack)
    assert lib.pmx_moe_reduce_allreduce_buffer_bytes(64, 4096, 0) == 16384 + 2 * (64 * 4096 // 8 + 256) * 32
    table = (C.c_void_p * 9)(*([16] * 9))
    assert lib.pmx_moe_reduce_allreduce(one, one, one, one, 4, 2, 64, 0, table, 0, 9, 1 << 30, 0, 0, 0, None) == -1  # > 8 ranks
    assert lib.pmx_moe_reduce_allreduce(one, one, one, one, 4, 2, 64, 0, table, 0, 2, 64, 0, 0, 0, None) == -4      # small buffers
    assert lib.pmx_moe_reduce_allreduce(one, one, one, one, 4, 2, 64, 0, table, 0, 2, 1 << 30, 7, 0, 0, None) == -1  # unknown algorithm
    assert lib.pmx_moe_set_programmatic_launch(1) in (0, 1)


def test_operators_refuse_cpu_tensors():
    import ppl.pmx_b200.torch_function as F
    x, s = torch.randn(4, 8), torch.randn(4, 8)
    w = torch.randn(8, 16, 8)
    off = torch.arange(9).clamp(max=4)
    for call in (lambda: F.moe_select(x, s, 8, 2),
                 lambda: F.moe_column_parallel_linear(x, off, w, None, None, 8, 8, 16, False),
                 lambda: F.moe_row_parallel_linear(x, off, w, None, None, 8, 8, 16, True),
                 lambda: F.moe_reduce(x.view(2, 2, 8), s[:2, :2], torch.zeros(2, 2, dtype=torch.long), 2),
                 lambda: F.swiglu(x), lambda: F.silu(x, x)):
        with pytest.raises(RuntimeError, match="no CPU fallback"):
            call()


def _graph_nodes(module, args):
    from torch.onnx._internal.torchscript_exporter import utils as U, _globals
    _globals.GLOBALS.export_onnx_opset_version = 11
    _globals.GLOBALS.in_onnx_export = True
    try:
        with U.exporter_context(module, torch.onnx.TrainingMode.EVAL, False):
            graph, _, _ = U._model_to_graph(module, args, do_constant_folding=False)
    finally:
        _globals.GLOBALS.in_onnx_export = False
    nodes = []
    for n in graph.nodes():
        if n.kind().startswith("opmx::"):
            attrs = {a: (n.f(a) if n.kindOf(a) == "f" else n.i(a)) for a in n.attributeNames()}
            nodes.append({"kind": n.kind(), "attrs": attrs, "n_inputs": len(list(n.inputs())),
                          "n_outputs": len(list(n.outputs()))})
    return nodes, graph


def test_onnx_export_matches_the_reference_graph():
    import ppl.pmx_b200.torch_function as F

    class M(torch.nn.Module):       # the module tests/golden/make_golden.py exported with the reference ops
        def __init__(s):
            super().__init__()
            s.wu = torch.nn.Parameter(torch.randn(8, 64, 32))
            s.wd = torch.nn.Parameter(torch.randn(8, 32, 32))
            s.bu = torch.nn.Parameter(torch.randn(8, 64))

        def forward(s, X, S):
            xe, ew, inv, off = F.moe_select(X, S, 8, 2)
            h = F.swiglu(F.moe_column_parallel_linear(xe, off, s.wu, s.bu, None, 8, 32, 64, False))
            y = F.moe_row_parallel_linear(h, off, s.wd, None, None, 8, 32, 32, True)
            return F.moe_reduce(y, ew, inv, 2)

    nodes, graph = _graph_nodes(M(), (torch.randn(4, 32), torch.randn(4, 8)))
    with open(os.path.join(ROOT, "tests", "golden", "onnx_block_graph.json")) as f:
        ref = json.load(f)["nodes"]
    assert nodes == ref
    # wiring: select's four outputs feed the linears (X, offsets) and the reduce (weights, permutation)
    by_kind = {n.kind(): n for n in graph.nodes() if n.kind().startswith("opmx::")}
    sel = list(by_kind["opmx::MoeSelect"].outputs())
    col_in = list(by_kind["opmx::MoeColumnParallelLinear"].inputs())
    red_in = list(by_kind["opmx::MoeReduce"].inputs())
    assert col_in[0] == sel[0] and col_in[1] == sel[3] and red_in[1] == sel[1] and red_in[2] == sel[2]


def test_rms_norm_exports_the_reference_node():
    import ppl.pmx_b200.torch_function as F

    class M(torch.nn.Module):
        def __init__(s):
            super().__init__()
            s.w = torch.nn.Parameter(torch.ones(32))

        def forward(s, X, S):
            y, h = F.skip_rms_norm(X, s.w, S, -1, 1e-6)
            return F.rms_norm(y, s.w, -1, 1e-5), h

    nodes, _ = _graph_nodes(M(), (torch.randn(4, 32), torch.randn(4, 32)))
    assert [n["kind"] for n in nodes] == ["opmx::RMSNorm", "opmx::RMSNorm"]
    assert nodes[0]["attrs"]["skip_term"] == 1 and nodes[0]["n_inputs"] == 3 and nodes[0]["n_outputs"] == 2
    assert nodes[1]["attrs"]["skip_term"] == 0 and nodes[1]["attrs"]["axis"] == -1
    assert abs(nodes[0]["attrs"]["eps"] - 1e-6) < 1e-12   # RMSNorm.py:9-10,33-39


def test_export_placeholders_have_output_shapes_and_dtypes():
    import ppl.pmx_b200.torch_function as F
    from torch.onnx._internal.torchscript_exporter import _globals
    _globals.GLOBALS.in_onnx_export = True
    try:
        x, s = torch.randn(2, 3, 16).half(), torch.randn(2, 3, 8).half()
        xe, ew, inv, off = F.moe_select(x, s, 8, 2)
        assert xe.shape == (2, 3, 2, 16) and ew.shape == (2, 3, 2) and inv.dtype == torch.int64 and off.shape == (9,)
        y = F.moe_column_parallel_linear(xe, off, torch.zeros(8, 24, 16).half(), None, None, 8, 16, 24, False)
        assert y.shape == (2, 3, 2, 24) and y.dtype == torch.float16
        assert F.swiglu(y).shape == (2, 3, 2, 12)
        z = F.moe_row_parallel_linear(F.swiglu(y), off, torch.zeros(8, 16, 12).half(), None, None, 8, 12, 16, True)
        assert F.moe_reduce(z, ew, inv, 2).shape == (2, 3, 16)
    finally:
        _globals.GLOBALS.in_onnx_export = False


def test_modules_have_the_reference_parameter_shapes():
    from ppl.pmx_b200.moe_layers import MoeColumnParallelLinear, MoeRowParallelLinear, MoeFeedForward
    col = MoeColumnParallelLinear(None, 8, 64, 256, bias_term=True, gather_output=False)
    row = MoeRowParallelLinear(None, 8, 128, 64, bias_term=False, input_is_parallel=True)
    assert col.weight.shape == (8, 256, 64) and col.bias.shape == (8, 256)      # ModelParallel.py:149-151
    assert row.weight.shape == (8, 64, 128) and row.bias is None                 # ModelParallel.py:184-188
    blk = MoeFeedForward(64, 128, 8, 2)
    assert sorted(blk.state_dict()) == ["gate.weight", "w2.weight", "wu.weight"]
    assert blk.wu.weight.shape == (8, 256, 64)
    with pytest.raises(AssertionError):
        class G:                                                                  # a 3-rank group
            def size(self):
                return 3
        MoeColumnParallelLinear(G(), 8, 64, 256)


def test_workloads_detie_and_algorithmic_work():
    from oracle import moe_oracle as orc
    from ppl.pmx_b200 import workloads as W
    for dt in (torch.float16, torch.bfloat16, torch.float32):
        s = torch.tensor([[1, 1, 1, 1, .5, 1, 1, 1], [0.0, -0.0, -1, -1, -2, -3, -4, -5]]).to(dt)
        before = s.clone()
        n = W.detie_(s)
        assert n > 0 and not orc.rows_with_ties(s.float().numpy(), 7).any()
        assert (s.float() - before.float()).abs().max() < 0.1
    sh = W.WORKLOADS["decode_t64"]
    x, wr, sc, nudges = W.make_activations(sh)
    assert x.shape == (64, 4096) and sc.shape == (64, 8) and sc.dtype == torch.float16
    assert not orc.rows_with_ties(sc.float().numpy(), 2).any()
    work = W.algorithmic_work(sh)
    assert abs(work["flops"] - 45.1e9) / 45.1e9 < 0.01           # 6*T*k*H*I
    assert abs(work["bytes"] - 2831e6) / 2831e6 < 0.01           # weights + materialised activations
    w8 = W.algorithmic_work(sh, tp_size=8)
    assert abs(w8["bytes"] - 358e6) / 358e6 < 0.02
    # shards are slices of the same full tensors (SplitModel.py:54-56)
    small = W.scaled(sh, H=32, I=64)
    full_u, full_d = W.make_expert_weights(small, "cpu")
    for r in range(2):
        u, d = W.make_expert_weights(small, "cpu", tp_rank=r, tp_size=2)
        assert torch.equal(u[:, :32], full_u[:, r * 32:(r + 1) * 32])
        assert torch.equal(u[:, 32:], full_u[:, 64 + r * 32:64 + (r + 1) * 32])
        assert torch.equal(d, full_d[:, :, r * 32:(r + 1) * 32])
    fg = W.WORKLOADS["finegrained_empty"]
    _, _, sc, _ = W.make_activations(fg)
    _, _, _, off = orc.moe_select(np.zeros((fg.T, 1), np.float32), sc.float().numpy(), fg.E, fg.k)
    assert int((np.diff(off) == 0).sum()) == 8


def test_patch_reference_rebinds_exactly_the_replaced_operators():
    """patch_reference() swaps the operators this package replaces into an imported OPMX
    `torch_function` module (the staged, unmodified reference), leaves every other
    attribute alone, and unpatch_reference() undoes it."""
    import oracle
    if oracle.ref_path() is None:
        pytest.skip("the OPMX reference is not staged (python oracle/make_ref.py)")
    import ppl.pmx_b200.torch_function as F
    from ppl.pmx_b200.moe_layers import patch_reference, unpatch_reference, PATCHED_NAMES
    opmx = oracle.import_reference()
    before, before_db = dict(vars(opmx)), dict(vars(opmx.dynamic_batching))
    saved = patch_reference(opmx)
    try:
        assert set(saved) == set(PATCHED_NAMES) == {
            "moe_select", "moe_column_parallel_linear", "moe_row_parallel_linear", "moe_reduce", "swiglu", "silu",
            "rms_norm", "skip_rms_norm", "linear", "column_parallel_linear", "row_parallel_linear",
            "dynamic_batching.multi_head_cache_attention"}
        for name, value in vars(opmx).items():
            if name in PATCHED_NAMES:
                assert value is getattr(F, name) and value is not before[name]
            else:
                assert value is before[name], f"{name} must not be touched"
        for name, value in vars(opmx.dynamic_batching).items():
            if name == "multi_head_cache_attention":
                assert value is not before_db[name]
            else:
                assert value is before_db[name], f"dynamic_batching.{name} must not be touched"
        with pytest.raises(ValueError):
            patch_reference(opmx, names=("multi_head_attention",))
    finally:
        unpatch_reference(opmx, saved)
    assert all(getattr(opmx, n) is before[n] for n in PATCHED_NAMES if "." not in n)
    assert opmx.dynamic_batching.multi_head_cache_attention is before_db["multi_head_cache_attention"]
