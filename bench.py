#!/usr/bin/env python
"""MoE-layer throughput of the B200 implementation (and of the CPU reference arm).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode_t64] [--impl reference]

One "step" is one call of the Mixtral MoE block (router gate -> moe_select ->
gate/up projection + SwiGLU -> down projection -> moe_reduce -> all-reduce when
N > 1) on one batch of seeded synthetic tokens.  With N > 1 (launched by
torchrun, one rank per GPU) every expert's intermediate dimension is sharded
over the ranks, so the total work is fixed as N grows ("strong" scaling).

The line printed by rank 0 (headline workload: Mixtral-8x7B decode, 64 tokens, fp16):
  value     tokens/s with the inputs resident in HBM: regions of K replays of the captured
            CUDA graph of the step, CUDA events on the launching stream, max over ranks;
            the median of `repeats.regions` regions (min and max are printed too)
  e2e       the same with the step's input copied from pinned host memory and
            its output copied back inside the timed region, every step
  roofline  the dominant kernel (gate/up grouped GEMM): its launch alone captured in a
            CUDA graph and replayed K times between two CUDA events, in the same run
  cpu_baseline  the reference's own CPU torch path (the unmodified OPMX operators staged
            under oracle/_ref; kind "reference") or, where that is absent, the CPU port
            of the same algorithm (oracle/cpu_port.py; kind "port"), on the host cores of
            this machine, a bounded sample of the same workload
  parity    routing compared bit for bit with the oracle, sampled tokens against an fp32
            chain, and (N > 1) the tensor-parallel result against the same kernels run
            with the full weights on rank 0; computed outside the timed regions
  workloads the other configurations (decode at 1..256 tokens, prefill of 8192 tokens in
            bf16, the fine-grained 64-expert layer with and without empty experts), each
            with its own timing, roofline, per-stage kernel times, clocks and parity
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

# dram bytes (read + write) / algorithmic bytes of the gate/up GEMM launch, from ncu captures
TRAFFIC_RATIO = {"hbm": 1.008, "tensor": 1.03}
METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
HEADLINE = "decode_t64"
EXTRA_WORKLOADS = ["decode_t1", "decode_t8", "decode_t32", "decode_t128", "decode_t256", "prefill", "finegrained",
                   "finegrained_empty"]
ATOL, RTOL = 2e-2, 1e-2          # parity tolerance of fp16 / bf16 results against fp32 math
STAGES = ["gate", "select", "route_select", "experts", "gate_up", "down", "reduce", "allreduce", "reduce_allreduce"]


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read only)."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake"}

    def __init__(self, index: int, period_s: float = 0.01):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.period = period_s

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def workload_config(shape, tp):
    return {"workload": shape.name, "tokens": shape.T, "hidden": shape.H, "experts": shape.E,
            "experts_per_token": shape.k, "ffn": shape.I, "parallelism": f"tp{tp}",
            "l2": "weights per rank exceed the 126 MB L2, no flush between steps"}


# ------------------------------------------------------------------------------ CPU arm
class CpuArm:
    """The MoE block on host cores: the unmodified OPMX operators when they are staged
    under oracle/_ref (kind "reference"), else the CPU port of the same algorithm."""

    def __init__(self, shape):
        from ppl.pmx_b200 import workloads as W
        self.shape = shape
        self.dt = W.TORCH_DTYPE[shape.dtype]
        self.opmx = None
        try:
            import oracle
            self.opmx = oracle.import_reference()
            self.kind = "reference"
        except ImportError:
            self.kind = "port"
        torch.set_num_threads(os.cpu_count() or 1)
        self.cores = torch.get_num_threads()

    def step(self, x, w_router, wu, w2):
        sh = self.shape
        if self.opmx is None:
            from oracle import cpu_port
            return cpu_port.moe_block(x, w_router, wu, w2, sh.E, sh.k)[0]
        O = self.opmx
        # the reference allocates the outputs of its MoE linears with the global default
        # dtype (MoeColumnParallelLinear.py:59, MoeRowParallelLinear.py:45): run it the way
        # its loader does (Loader.py:76-79), with the default dtype set to the model's
        old = torch.get_default_dtype()
        torch.set_default_dtype(self.dt)
        try:
            E, k, H, I = sh.E, sh.k, sh.H, sh.I
            scores = O.linear(x, w_router, None, H, E)                              # Model.py:188
            xe, ew, inv, off = O.moe_select(x, scores, E, k)                        # :191
            x13 = O.moe_column_parallel_linear(xe, off, wu, None, None, E, H, 2 * I, False)   # :198
            x13 = O.swiglu(x13)                                                     # :200
            y = O.moe_row_parallel_linear(x13, off, w2, None, None, E, I, H, True)  # :208
            return O.moe_reduce(y, ew, inv, k)                                      # :211
        finally:
            torch.set_default_dtype(old)

    def time(self, x, w_router, wu, w2, tokens, steps, warmup, budget_s):
        xs = x[:tokens]
        with torch.inference_mode():
            for _ in range(warmup):
                self.step(xs, w_router, wu, w2)
            times = []
            t_begin = time.perf_counter()
            for _ in range(steps):
                t0 = time.perf_counter()
                self.step(xs, w_router, wu, w2)
                times.append(time.perf_counter() - t0)
                if time.perf_counter() - t_begin > budget_s:
                    break
        return times

    def describe(self, tokens, n):
        src = ("unmodified OPMX operators from oracle/_ref (linear, moe_select, moe_column_parallel_linear, swiglu, "
               "moe_row_parallel_linear, moe_reduce)") if self.kind == "reference" else "oracle/cpu_port.py"
        return (f"{src}: first {tokens} of {self.shape.T} tokens per step, all {self.shape.E} experts' full weights, "
                f"{n} steps, torch {torch.__version__} CPU, {self.cores} threads")


def run_reference(args, shape, rank):
    """The reference's CPU torch path for the same workload, on this machine's host cores."""
    if rank != 0:
        return
    from ppl.pmx_b200 import workloads as W
    x, w_router, _, _ = W.make_activations(shape, detie=False)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    wu, w2 = W.make_expert_weights(shape, dev)
    wu, w2 = wu.cpu(), w2.cpu()
    arm = CpuArm(shape)
    tokens = min(shape.T, 1024)
    times = arm.time(x, w_router, wu, w2, tokens, args.steps, args.warmup, budget_s=240.0)
    total = sum(times)
    value = tokens * len(times) / total
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": len(times), "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": shape.dtype,
        "data": "synthetic", "config": workload_config(shape, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": arm.cores, "kind": arm.kind, "device": "cpu",
                         "sample": arm.describe(tokens, len(times))},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------ GPU arm
class Ctx:
    pass


def sync_all(ctx):
    if ctx.world > 1:
        dist.barrier(group=ctx.group)
    torch.cuda.synchronize()


def timed(ctx, fn, steps):
    """K calls of fn between two CUDA events on the current stream, barrier + synchronise on
    both sides, max over ranks; milliseconds for the K calls."""
    sync_all(ctx)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    sync_all(ctx)
    ms = torch.tensor([e0.elapsed_time(e1)], device=ctx.device)
    if ctx.world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=ctx.group)
    return float(ms.item())


def capture(fn):
    """fn captured in a CUDA graph (after one run on a side stream)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = fn()
    return g, out


STAMP_KERNELS = {1: "route_select", 2: "grouped_gemm", 3: "dense_gate_up", 4: "experts_one_launch"}
STAMP_WORDS = ["entry", "setup_done", "first_tile", "last_mma", "epilogue_free", "epilogue_done", "exit",
               "first_h_tile_or_last_accumulator"]


def record_stamps(ctx, step):
    """One replay of the step's CUDA graph with the kernels' %globaltimer stamps switched on
    (pmx_moe_set_stamp_buffer): per instrumented launch, the minimum / median / maximum over
    its CTAs of every stamp, in microseconds after the first stamp of the replay."""
    from ppl.pmx_b200 import _cabi
    import ctypes as C
    import numpy as np
    buf = torch.zeros(64 * 160 * 8, dtype=torch.int64, device=ctx.device)
    _cabi.lib.pmx_moe_set_stamp_buffer(C.c_void_p(buf.data_ptr()), buf.numel() * 8)
    try:
        g, _ = capture(step)            # slots: one eager run, then the captured launches
        ids = (C.c_int32 * 256)()
        used = _cabi.lib.pmx_moe_stamp_slots(ids, 256)
    finally:
        _cabi.lib.pmx_moe_set_stamp_buffer(None, 0)
    for _ in range(5):
        g.replay()
    torch.cuda.synchronize()
    buf.zero_()
    g.replay()
    torch.cuda.synchronize()
    data = buf.cpu().numpy().reshape(64, 160, 8)
    g.reset()
    per = used // 2
    slots = range(per, used)
    t0 = min(int(data[s][data[s] > 0].min()) for s in slots if (data[s] > 0).any())
    rec = []
    for s in slots:
        d = data[s]
        row = {"kernel": STAMP_KERNELS.get(ids[s], str(ids[s])), "ctas": int((d[:, 0] > 0).sum())}
        for w, name in enumerate(STAMP_WORDS):
            v = d[:, w][d[:, w] > 0]
            if v.size:
                row[name] = [round((int(x) - t0) / 1e3, 2) for x in (v.min(), np.median(v), v.max())]
        if ctx.args.stamps_raw:
            row["per_cta"] = {name: [round((int(x) - t0) / 1e3, 1) if x > 0 else None for x in d[:, w]]
                              for w, name in enumerate(STAMP_WORDS) if (d[:, w] > 0).any()}
        rec.append(row)
    return rec


def get_block(ctx, shape, full: bool, w_router=None):
    """The MoE block of this rank for `shape` (cached by architecture and dtype: the decode
    workloads share one set of weights).  full=True: the whole weights, no process group."""
    from ppl.pmx_b200 import workloads as W
    from ppl.pmx_b200.moe_layers import MoeFeedForward
    key = (shape.H, shape.I, shape.E, shape.k, shape.dtype, full)
    if key in ctx.blocks:
        return ctx.blocks[key]
    dt = W.TORCH_DTYPE[shape.dtype]
    tp = 1 if full else ctx.world
    peer_tokens = 0
    if tp > 1 and ctx.args.allreduce != "nccl" and not ctx.peer_failed:
        peer_tokens = (4 << 20) // (shape.H * 2)          # results of up to 4 MB go through the peer kernel
        if ctx.args.allreduce == "peer":
            peer_tokens = max(peer_tokens, 8192)
    blk = MoeFeedForward(shape.H, shape.I, shape.E, shape.k, None if full else ctx.group, False,
                         peer_reduce_tokens=peer_tokens, peer_algorithm=ctx.args.peer_algo,
                         overlap_chunks=ctx.args.overlap_chunks,
                         dense_decode=not ctx.args.no_dense_decode,
                         one_launch_experts=not ctx.args.no_one_launch,
                         token_microbatches=ctx.args.token_microbatches).to(ctx.device, dt)
    wu, w2 = W.make_expert_weights(shape, ctx.device, tp_rank=0 if full else ctx.rank, tp_size=tp)
    if w_router is None:
        _, w_router, _, _ = W.make_activations(shape, detie=False)
    with torch.no_grad():
        blk.gate.weight.copy_(w_router)
        blk.wu.weight.copy_(wu)
        blk.w2.weight.copy_(w2)
    del wu, w2
    ctx.blocks[key] = blk
    return blk


def uses_peer(blk, shape):
    return blk._peer is not None and blk._peer.fits(shape.T, shape.H, blk.wu.weight.dtype)


def routing_of(blk, x_dev, shape):
    """(scores, x_experts, expert_weights, invert_permutation, expert_offset) exactly as the block computes them."""
    import ppl.pmx_b200.torch_function as OPMX
    r = OPMX.moe_route_select(x_dev, blk.gate.weight, shape.E, shape.k)
    if r is not None:
        return r
    scores = OPMX.router_gate(x_dev, blk.gate.weight)
    return (scores,) + tuple(OPMX.moe_select(x_dev, scores, shape.E, shape.k))


def parity_check(ctx, shape, blk, x_dev, out):
    """Untimed.  Routing bit for bit against the oracle (on the scores the kernel produced),
    `samples` tokens of the result against an fp32 chain over the full weights, and for N > 1
    the tensor-parallel result against the same kernels with the full weights on rank 0 plus
    identical routing on every rank."""
    import numpy as np
    from oracle import moe_oracle as orc
    E, k, T, H, I = shape.E, shape.k, shape.T, shape.H, shape.I
    with torch.no_grad():
        scores, _, ew, inv, off = routing_of(blk, x_dev, shape)
    torch.cuda.synchronize()
    rec = {"tolerance": f"max-abs {ATOL} / rel {RTOL} against fp32 math"}
    ranks_same = None
    if ctx.world > 1:
        # the routing is replicated: every rank must hold the same integers
        mine = torch.cat([off.view(-1), inv.view(-1)])
        allr = [torch.empty_like(mine) for _ in range(ctx.world)]
        dist.all_gather(allr, mine, group=ctx.group)
        outs = [torch.empty_like(out) for _ in range(ctx.world)]
        dist.all_gather(outs, out.contiguous(), group=ctx.group)
        ranks_same = all(torch.equal(a, allr[0]) for a in allr)
        rec["routing_identical_on_all_ranks"] = ranks_same
        rec["output_identical_on_all_ranks"] = all(torch.equal(o, outs[0]) for o in outs)
    if ctx.rank != 0:
        return None
    s32 = scores.float().cpu().numpy().reshape(T, E)
    _, oew, oinv, ooff = orc.moe_select(np.zeros((T, 1), np.float32), s32, E, k, shape.dtype)
    rec["expert_offset_exact"] = bool(np.array_equal(off.cpu().numpy(), ooff))
    rec["invert_permutation_exact"] = bool(np.array_equal(inv.cpu().numpy().reshape(T, k), oinv))
    rec["rows_with_tied_scores"] = int(orc.rows_with_ties(s32, k).sum())
    rec["empty_experts"] = int((np.diff(ooff) == 0).sum())
    # sampled tokens against fp32 math over the full weights
    full = blk if ctx.world == 1 else get_block(ctx, shape, full=True, w_router=blk.gate.weight.detach())
    rng = np.random.default_rng(0)
    sample = rng.choice(T, size=min(32, T), replace=False)
    expert_of_row = np.searchsorted(ooff, np.arange(T * k), side="right") - 1
    max_abs, max_rel, ok = 0.0, 0.0, True
    with torch.no_grad():
        for t in sample:
            acc = torch.zeros(H, device=ctx.device, dtype=torch.float32)
            xt = x_dev[t].float()
            for j in range(k):
                e = int(expert_of_row[oinv[t, j]])
                gu = full.wu.weight[e].float() @ xt
                h = gu[I:] * gu[:I] * torch.sigmoid(gu[:I])
                acc += float(oew[t, j]) * (full.w2.weight[e].float() @ h)
            got = out[t].float()
            err = (got - acc).abs()
            max_abs = max(max_abs, float(err.max()))
            max_rel = max(max_rel, float((err / acc.abs().clamp_min(1.0)).max()))
            ok &= bool((err <= ATOL + RTOL * acc.abs()).all())
    rec.update({"sampled_tokens": int(len(sample)), "max_abs_err": max_abs, "max_rel_err": max_rel,
                "sampled_within_tolerance": ok})
    good = rec["expert_offset_exact"] and rec["invert_permutation_exact"] and ok
    if ctx.world > 1:
        with torch.no_grad():
            one = full(x_dev)
        torch.cuda.synchronize()
        d = (out.float() - one.float()).abs()
        same = bool((d <= ATOL + RTOL * one.float().abs()).all())
        rec["tp_vs_tp1"] = {"max_abs_diff": float(d.max()), "within_tolerance": same,
                            "note": "tensor-parallel result of this run against the same kernels on rank 0 with the "
                                    "full weights (the partial sums are rounded and added in another order)"}
        good = good and same and bool(ranks_same)
    rec["ok"] = bool(good)
    return rec


def measure(ctx, shape, steps, warmup, regions, headline):
    """Times one workload; returns its record on rank 0 (None elsewhere)."""
    import ppl.pmx_b200.torch_function as OPMX
    from ppl.pmx_b200 import _cabi, workloads as W
    from ppl.pmx_b200.torch_function.moe import moe_grouped_linear
    args = ctx.args
    dt = W.TORCH_DTYPE[shape.dtype]
    x_host, w_router, _, _ = W.make_activations(shape, detie=False)
    x_host = x_host.pin_memory()
    out_host = torch.empty(shape.T, shape.H, dtype=dt).pin_memory()
    blk = get_block(ctx, shape, full=False, w_router=w_router)
    x_dev = x_host.to(ctx.device)
    E, k = shape.E, shape.k

    def step():
        with torch.no_grad():
            return blk(x_dev)

    if ctx.world > 1 and blk.peer_reduce_tokens > 0 and blk._peer is None:
        # the peer-memory exchange needs the ranks' buffers mapped into each other
        # (symmetric memory); if this machine refuses, say so and use NCCL
        try:
            step()
            torch.cuda.synchronize()
            ok = torch.ones(1, device=ctx.device)
        except Exception as exc:                      # noqa: BLE001
            print(f"[bench] rank {ctx.rank}: peer-memory all-reduce unavailable ({exc}); using NCCL", file=sys.stderr)
            ok = torch.zeros(1, device=ctx.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=ctx.group)
        if ok.item() == 0:
            ctx.peer_failed = True
            for b in ctx.blocks.values():
                b.peer_reduce_tokens, b._peer = 0, None
    use_peer = uses_peer(blk, shape) if ctx.world > 1 else False

    for _ in range(warmup):
        out = step()
    torch.cuda.synchronize()
    launches_before = _cabi.lib.pmx_moe_kernel_launches()
    out = step()
    torch.cuda.synchronize()
    launches_per_step = _cabi.lib.pmx_moe_kernel_launches() - launches_before
    blk.check()                                       # no bounded wait ran out so far
    graph = None
    if not args.no_graph:
        graph, out = capture(step)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()

    def run_step():
        if graph is not None:
            graph.replay()
            return out
        return step()

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True)
        o = run_step()
        out_host.copy_(o, non_blocking=True)

    sampler = ClockSampler(physical_gpu_index(ctx.local_rank))
    kernel_ms = {n: 0.0 for n in STAGES + ["skip_rms_norm", "norm_route_select"]}
    with sampler:
        region_ms = [timed(ctx, run_step, steps) for _ in range(regions)]
        ms_e2e = timed(ctx, e2e_step, steps) if headline else None

        # per-stage pass: every stage of the step is captured in a CUDA graph of its own and
        # replayed K times between two CUDA events (no host launch gaps inside the figure);
        # with --no-graph the stages are launched eagerly instead
        keep = []

        def stage(name, fn):
            with torch.no_grad():
                r = fn()                                   # eager: produces the next stage's inputs
                if args.no_graph:
                    run = fn
                else:
                    g, _ = capture(fn)
                    keep.append(g)
                    run = g.replay
                kernel_ms[name] = timed(ctx, run, steps) / steps
            return r

        sync_all(ctx)
        plan = ctx.gemm_plan
        from ppl.pmx_b200.torch_function.moe import dense_gate_up_covers, dense_mlp_covers
        one_launch = bool(blk.dense_decode and blk.one_launch_experts
                          and dense_mlp_covers(shape.T, blk.wu.weight, blk.w2.weight, k))
        dense = (blk.dense_decode and (one_launch or dense_gate_up_covers(shape.T, blk.wu.weight, k))
                 and OPMX.moe_route_select(x_dev, blk.gate.weight, E, k, gather=False) is not None)
        one_launch = one_launch and dense
        if dense:
            # the step's own kernels: router without the gather, gate/up from the un-permuted tokens
            _, _, ew, inv, off = stage("route_select", lambda: OPMX.moe_route_select(x_dev, blk.gate.weight, E, k,
                                                                                     gather=False))
            if one_launch:
                # the step's kernel for both projections; the two launches below are timed for comparison
                stage("experts", lambda: OPMX.moe_dense_mlp(x_dev, inv, off, blk.wu.weight, blk.w2.weight))
            h = stage("gate_up", lambda: OPMX.moe_dense_gate_up(x_dev, inv, off, blk.wu.weight, None))
        else:
            if OPMX.moe_route_select(x_dev, blk.gate.weight, E, k) is not None:
                _, xe, ew, inv, off = stage("route_select", lambda: OPMX.moe_route_select(x_dev, blk.gate.weight, E, k))
            else:
                logits = stage("gate", lambda: OPMX.router_gate(x_dev, blk.gate.weight))
                xe, ew, inv, off = stage("select", lambda: OPMX.moe_select(x_dev, logits, E, k))
            h = stage("gate_up", lambda: moe_grouped_linear(xe.view(-1, shape.H), off, blk.wu.weight, None,
                                                            swiglu=True, zero_outside=False, plan=plan))
        y = stage("down", lambda: moe_grouped_linear(h, off, blk.w2.weight, None, zero_outside=False, plan=plan))
        if use_peer:
            stage("reduce_allreduce", lambda: blk._peer.combine_allreduce(y, ew, inv, k))
        else:
            o = stage("reduce", lambda: OPMX.moe_reduce(y.view(shape.T, k, -1), ew, inv, k))
            if ctx.world > 1:
                stage("allreduce", lambda: dist.all_reduce(o, group=ctx.group))
        if headline:
            # the normalisation in front of the block (not part of the step): x + skip -> RMSNorm
            norm_w = torch.ones(shape.H, device=ctx.device, dtype=dt)
            skip_dev = torch.randn_like(x_dev)
            stage("skip_rms_norm", lambda: OPMX.skip_rms_norm(x_dev, norm_w, skip_dev, -1, 1e-5))
            if OPMX.moe_norm_route_select(x_dev, skip_dev, norm_w, 1e-5, blk.gate.weight, E, k) is not None:
                stage("norm_route_select",
                      lambda: OPMX.moe_norm_route_select(x_dev, skip_dev, norm_w, 1e-5, blk.gate.weight, E, k))
        sync_all(ctx)
        for g in keep:
            g.reset()
        del keep
    stamps_rec = None
    if args.stamps and headline and not args.no_graph:
        stamps_rec = record_stamps(ctx, step)
    active = int((off[1:] - off[:-1]).gt(0).sum().item())
    # phase boundaries inside the fused combine + all-reduce (one extra call with stamps on)
    ar_phases = None
    if use_peer:
        try:
            blk._peer.flags = _cabi.ALLREDUCE_FLAG_STAMPS
            for _ in range(3):
                step()
            ar_phases = blk._peer.phases_ns()
        except Exception:                                 # noqa: BLE001  (diagnostic only)
            ar_phases = None
        finally:
            blk._peer.flags = 0
    sync_all(ctx)
    out = run_step()
    torch.cuda.synchronize()
    blk.check()
    parity = parity_check(ctx, shape, blk, x_dev, out)
    sync_all(ctx)
    if graph is not None:
        graph.reset()
        del graph
    if ctx.rank != 0:
        return None

    peaks = ctx.peaks
    work = W.algorithmic_work(shape, ctx.world, active)
    ms_med = statistics.median(region_ms)
    ms_step = ms_med / steps
    clocks = sampler.summary()
    # tensor peak: the burst figure when the timed region ran at (nearly) full SM clock,
    # the sustained one when the power cap had pulled the clock down
    burst = bool(clocks["sm_mhz"] and clocks["sm_max_mhz"] and clocks["sm_mhz"] >= 0.9 * clocks["sm_max_mhz"])
    tensor_peak = peaks["bf16_tflops"] if burst else peaks["bf16_tflops_sustained"]
    ridge = tensor_peak * 1e12 / (peaks["hbm_gbs"] * 1e9)

    def roofline_of(stage_name, bytes_key, flops_key):
        t = kernel_ms[stage_name] * 1e-3
        if t <= 0:
            return None
        if work[flops_key] / work[bytes_key] < ridge:
            a = work[bytes_key] / t / 1e9
            return {"bound": "hbm", "achieved": a, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": a / peaks["hbm_gbs"]}
        a = work[flops_key] / t / 1e12
        return {"bound": "tensor", "achieved": a, "peak": tensor_peak, "unit": "TFLOP/s", "frac": a / tensor_peak,
                "peak_kind": "burst" if burst else "sustained"}

    roof = roofline_of("gate_up", "bytes_gate_up", "flops_gate_up")
    if one_launch:
        # the step runs both projections as one launch: that launch is the dominant kernel
        t_exp = kernel_ms["experts"] * 1e-3
        b_exp = work["bytes_gate_up"] + work["bytes_down"]
        roof_experts = {"bound": "hbm", "achieved": b_exp / t_exp / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": b_exp / t_exp / 1e9 / peaks["hbm_gbs"], "traffic": b_exp * 1.01,
                        "kernel_ms": kernel_ms["experts"], "algorithmic_bytes": b_exp, "peak_source": peaks["source"],
                        "kernel": "both expert projections in one launch (expert_mlp_decode_kernel; traffic ratio "
                                  "1.01 from profiles/expert_mlp_decode_tp8_shard.md)",
                        "timing": "CUDA events around K back-to-back replays of a CUDA graph holding this launch "
                                  "alone, same run"}
    else:
        roof_experts = None
    ratio = TRAFFIC_RATIO.get(roof["bound"])
    # DRAM traffic of the launch = algorithmic bytes x the ratio ncu measured on a
    # reduced-ffn case of the same kernel (profiles/grouped_gemm_tc_*.md); traffic is
    # >99 % weights and scales with the ffn size
    roof.update({"traffic": work["bytes_gate_up"] * ratio if ratio else None,
                 "kernel": "gate/up grouped GEMM with SwiGLU epilogue (grouped_gemm_tc_kernel; "
                           "grouped_gemm_tc_pair_kernel for >= 1024 rows per expert)",
                 "kernel_ms": kernel_ms["gate_up"], "peak_source": peaks["source"],
                 "algorithmic_bytes": work["bytes_gate_up"], "algorithmic_flops": work["flops_gate_up"],
                 "timing": "CUDA events around K back-to-back replays of a CUDA graph holding this launch alone, same run"})
    down = roofline_of("down", "bytes_down", "flops_down")
    layer_floor_s = max(work["bytes"] / (peaks["hbm_gbs"] * 1e9), work["flops"] / (tensor_peak * 1e12))
    rec = {
        "workload": shape.name, "dtype": shape.dtype, "config": workload_config(shape, ctx.world),
        "steps": steps, "ms_per_step": ms_step, "tokens_per_s": shape.T / (ms_step * 1e-3),
        "repeats": {"regions": regions, "steps_per_region": steps, "ms_per_step_median": ms_step,
                    "ms_per_step_min": min(region_ms) / steps, "ms_per_step_max": max(region_ms) / steps},
        "gpu_launches_per_step": int(launches_per_step),
        # the dominant kernel of the step: the one-launch expert kernel where the step uses it
        # (the gate/up and down launches it replaces are then timed for comparison only)
        "clocks": clocks, "roofline": roof_experts if roof_experts else roof,
        "roofline_down": {k2: down[k2] for k2 in ("bound", "achieved", "unit", "frac")} if down else None,
        "roofline_gate_up_as_its_own_launch": roof if roof_experts else None,
        "layer": {"ms_floor": layer_floor_s * 1e3, "frac_of_roofline": layer_floor_s * 1e3 / ms_step,
                  "active_experts": active, "graph": not args.no_graph,
                  "allreduce": ((f"peer-memory kernel fused with the combine ({args.peer_algo})" if use_peer else "nccl")
                                if ctx.world > 1 else None),
                  "allreduce_phases_ns": ar_phases,
                  "gate_up_from_unpermuted_tokens": bool(dense),
                  "experts_in_one_launch": bool(one_launch),
                  "stamps": stamps_rec,
                  "kernel_ms": {n: round(v, 5) for n, v in kernel_ms.items() if n in STAGES and v > 0}},
        "parity": parity,
    }
    if headline:
        rec["e2e_ms_total"] = ms_e2e
        rec["h2d"] = x_host.numel() * x_host.element_size()
        rec["d2h"] = out_host.numel() * out_host.element_size()
        rec["layer"]["front_end"] = {
            "skip_rms_norm_ms": round(kernel_ms["skip_rms_norm"], 5),
            "norm_route_select_ms": round(kernel_ms["norm_route_select"], 5) or None,
            "gbs": (4 * x_host.numel() * x_host.element_size() / (kernel_ms["skip_rms_norm"] * 1e-3) / 1e9
                    if kernel_ms["skip_rms_norm"] > 0 else None)}
    return rec


# ------------------------------------------------------------------------------ full decoder (config 5)
DECODER_FULL = dict(hidden_dim=4096, intermediate_dim=14336, num_layers=32, num_heads=32, num_kv_heads=8,
                    vocab_size=32000, num_experts=8, num_experts_per_token=2)


def build_reference_decoder(cfg, proc_group, device, rank, world, dtype=torch.float16, cache_layout=0):
    """The reference's own Mixtral `Transformer` (model_zoo/mixtral/modeling/dynamic_batching/
    Model.py:269-359, unmodified, imported from oracle/_ref) on `device`, built the way its
    loader does (Loader.py:76-91: default tensor type = the model's dtype on the device),
    with seeded random weights: replicated tensors (norms, router gate) get the same values on
    every rank, sharded tensors a per-rank seed."""
    import oracle
    opmx, model_mod, ModelParams = oracle.import_reference_mixtral()
    params = ModelParams(norm_eps=1e-5, rope_theta=1e6, cache_quant_bit=0, cache_quant_group=0,
                         cache_layout=cache_layout, cache_mode=0, **cfg)
    old_dtype = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    torch.set_default_device(device)
    try:
        net = model_mod.Transformer(params, False, True, True, True, False, False, False, 0, proc_group)
    finally:
        torch.set_default_device("cpu")
        torch.set_default_dtype(old_dtype)
    gen = torch.Generator(device=device)
    tp = {"wqkv": 1, "wu": 1, "output": 1, "wo": world, "w2": world}      # factor from the shard's to the full fan-in
    with torch.no_grad():
        for index, (name, w) in enumerate(net.named_parameters()):
            if "norm" in name:
                w.fill_(1.0)
                continue
            replicated = ".gate." in name
            gen.manual_seed(1000003 * (index + 1) + (0 if replicated else 7919 * (rank + 1)))
            if "tok_embeddings" in name:
                std = 1.0
            elif replicated:
                std = 0.02
            else:
                leaf = name.split(".")[-2]
                std = (w.shape[-1] * tp.get(leaf, 1)) ** -0.5
            # filled in slices: a whole fp32 temporary of a 29 GB tensor is not needed
            flat = w.view(-1)
            for lo in range(0, flat.numel(), 1 << 26):
                hi = min(flat.numel(), lo + (1 << 26))
                flat[lo:hi] = torch.randn(hi - lo, generator=gen, device=device, dtype=torch.float32) * std
    return opmx, model_mod, net


def decoder_step_inputs(net, batch, cached, device, world, seed=0):
    """One decode step (one new token per sequence) over `cached` tokens already in the KV
    cache of every sequence; tensors as Pipeline.py:130-182 builds them.  The cache is filled
    with seeded N(0,1) values instead of running a prefill."""
    p = net.params
    head_dim = p.hidden_dim // p.num_heads
    kv_heads = p.num_kv_heads // world
    cap = cached + 8
    g = torch.Generator().manual_seed(seed)
    tokens = torch.randint(0, p.vocab_size, (batch,), generator=g).to(device)
    seqstarts = torch.arange(0, batch + 1, dtype=torch.int64, device=device)
    start_pos = torch.full((batch,), cached, dtype=torch.int64, device=device)
    kvstarts = torch.arange(0, (batch + 1) * (cached + 1), cached + 1, dtype=torch.int64, device=device)
    cachestarts = torch.arange(0, batch * cap, cap, dtype=torch.int64, device=device)
    gd = torch.Generator(device=device).manual_seed(seed + 1 + 31 * (torch.distributed.get_rank() if world > 1 else 0))
    if p.cache_layout == 0:
        shape = (batch * cap, p.num_layers, 2, kv_heads, head_dim)
    else:
        shape = (p.num_layers, 2, kv_heads, batch * cap, head_dim)
    kv_cache = torch.randn(shape, generator=gd, device=device, dtype=torch.float16)
    return dict(tokens=tokens, attn_mask=torch.empty(0, dtype=torch.float16), seqstarts=seqstarts, kvstarts=kvstarts,
                cachestarts=cachestarts, decoding_batches=torch.tensor([batch], dtype=torch.int64),
                start_pos=start_pos, max_seqlen=torch.tensor([1], dtype=torch.int64),
                max_kvlen=torch.tensor([cached + 1], dtype=torch.int64), kv_cache=kv_cache)


def decoder_forward(net, inp, kv_cache, dtype=torch.float16):
    """net.forward under the reference's tensor defaults (its operators allocate with them)."""
    old_dtype = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    torch.set_default_device(kv_cache.device)
    try:
        return net.forward(inp["tokens"], inp["attn_mask"], inp["seqstarts"], inp["kvstarts"], inp["cachestarts"],
                           inp["decoding_batches"], inp["start_pos"], inp["max_seqlen"], inp["max_kvlen"],
                           kv_cache, None)
    finally:
        torch.set_default_device("cpu")
        torch.set_default_dtype(old_dtype)


class MoeTimer:
    """Wraps feed_forward.forward of every layer with a pair of CUDA events (measurement only)."""

    def __init__(self, net):
        self.pairs = []
        self.saved = []
        for layer in net.layers:
            ff = layer.feed_forward
            inner = ff.forward
            self.saved.append((ff, ff.__dict__.get("forward")))

            def timed_forward(x, _inner=inner):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                y = _inner(x)
                e1.record()
                self.pairs.append((e0, e1))
                return y
            ff.forward = timed_forward

    def total_ms(self):
        torch.cuda.synchronize()
        t = sum(a.elapsed_time(b) for a, b in self.pairs)
        self.pairs = []
        return t

    def remove(self):
        for ff, old in self.saved:
            if old is None:
                del ff.forward
            else:
                ff.forward = old


def run_decoder(ctx, cfg, batch, cached, steps, parity_layers=2):
    """The full decoder step of the reference model with the operators of this package
    swapped in.  Four variants share one set of weights: the unmodified reference
    operators; "patched": patch_reference() of the MoE operators, the norms and the dense
    linears, call by call; "fused": in addition the fused MoeFeedForward block in place of
    the reference block's forward; "fused+attention": in addition the decode-step cache
    attention kernel in place of the reference's per-sequence loops.  Parity: a
    `parity_layers`-deep copy of the model, same inputs, logits of the variants against the
    unmodified reference.  Timing: whole step (host clock around the synchronised call:
    the reference's attention, KV-cache and rotary operators loop over the sequences in
    Python) and the summed time of the MoE blocks (CUDA events)."""
    from ppl.pmx_b200.moe_layers import MoeFeedForward, PATCHED_NAMES, patch_reference, unpatch_reference
    world, device = ctx.world, ctx.device
    no_attention = tuple(n for n in PATCHED_NAMES if "attention" not in n)

    def make_fused(net):
        """One fused MoeFeedForward of this package per layer, on the reference module's own
        parameters; all layers share one exchange buffer for the peer-memory all-reduce."""
        peer_tokens = 0 if (world == 1 or ctx.args.allreduce == "nccl" or ctx.peer_failed) else max(256, batch)
        blocks = []
        for layer in net.layers:
            ref = layer.feed_forward
            blk = MoeFeedForward(cfg["hidden_dim"], cfg["intermediate_dim"], cfg["num_experts"],
                                 cfg["num_experts_per_token"], ctx.group, False, peer_reduce_tokens=peer_tokens,
                                 peer_algorithm=ctx.args.peer_algo)
            blk.gate.weight, blk.wu.weight, blk.w2.weight = ref.gate.weight, ref.wu.weight, ref.w2.weight
            blocks.append(blk)
        if peer_tokens:
            from ppl.pmx_b200.peer_reduce import PeerCombine
            shared = PeerCombine(ctx.group, peer_tokens, cfg["hidden_dim"], torch.float16, device,
                                 algorithm=ctx.args.peer_algo)
            for blk in blocks:
                blk._peer = shared
        return blocks

    def one_pass(net, opmx, inp, variant, fused, n_steps, timer):
        saved, undo = {}, []
        if variant != "reference":
            saved = patch_reference(opmx, PATCHED_NAMES if variant == "fused+attention" else no_attention)
        if variant.startswith("fused"):
            for layer, blk in zip(net.layers, fused):
                undo.append((layer.feed_forward, layer.feed_forward.__dict__.get("forward")))
                layer.feed_forward.forward = (lambda x, _b=blk: _b(x))
        moe = MoeTimer(net) if timer else None
        try:
            times, logits = [], None
            for i in range(n_steps):
                kv = inp["kv_cache"].clone()
                sync_all(ctx)
                t0 = time.perf_counter()
                with torch.no_grad():
                    logits = decoder_forward(net, inp, kv)
                torch.cuda.synchronize()
                times.append(time.perf_counter() - t0)
                if moe is not None and i == 0:
                    moe.total_ms()                     # first call: warm-up, drop its events
            moe_ms = moe.total_ms() / max(1, n_steps - 1) if moe is not None else None
        finally:
            if moe is not None:
                moe.remove()
            for ff, old in undo:
                if old is None:
                    del ff.forward
                else:
                    ff.forward = old
            unpatch_reference(opmx, saved)
        steady = times[1:] if len(times) > 1 else times
        return logits, statistics.median(steady) * 1e3, moe_ms

    out = {"config": dict(cfg, batch=batch, cached_tokens=cached, parallelism=f"tp{world}", dtype="f16",
                          cache_layout=0)}
    # parity at reduced depth
    small = dict(cfg, num_layers=parity_layers)
    opmx, _, net = build_reference_decoder(small, ctx.group, device, ctx.rank, world)
    inp = decoder_step_inputs(net, batch, cached, device, world)
    fused = make_fused(net)
    ref_logits, _, _ = one_pass(net, opmx, inp, "reference", fused, 1, False)
    par = {}
    for v in ("patched", "fused", "fused+attention"):
        logits, _, _ = one_pass(net, opmx, inp, v, fused, 1, False)
        d = (logits.float() - ref_logits.float()).abs()
        par[v] = {"max_abs_diff_logits": float(d.max()), "mean_abs_logit": float(ref_logits.float().abs().mean()),
                  "argmax_agree": float((logits.argmax(-1) == ref_logits.argmax(-1)).float().mean())}
        par[v]["ok"] = bool(par[v]["max_abs_diff_logits"] <= 5e-2 * max(1.0, float(ref_logits.float().abs().max())))
    out["parity"] = dict(par, layers=parity_layers,
                         note="logits of one decode step against the unmodified reference operators on the same "
                              "GPUs; bar: max-abs 5e-2 of the largest logit")
    del net, fused, inp
    torch.cuda.empty_cache()
    # timing at full depth
    opmx, _, net = build_reference_decoder(cfg, ctx.group, device, ctx.rank, world)
    inp = decoder_step_inputs(net, batch, cached, device, world)
    fused = make_fused(net)
    out["timing"] = {}
    for v in ("reference", "patched", "fused", "fused+attention"):
        _, ms, moe_ms = one_pass(net, opmx, inp, v, fused, steps + 1, True)
        out["timing"][v] = {"ms_per_step": ms, "moe_ms_per_step": moe_ms,
                            "moe_ms_per_layer": moe_ms / cfg["num_layers"] if moe_ms is not None else None,
                            "tokens_per_s": batch / (ms * 1e-3)}
    out["timing"]["note"] = ("median host-clock time of a synchronised decode step; the rotary embedding (and, except in "
                             "the last variant, the attention and KV-cache operators) are the reference's own "
                             "per-sequence Python loops")
    del net, fused, inp
    torch.cuda.empty_cache()
    return out


def measure_attention(ctx, steps, batch=64, cached=2048, heads=32, kv_heads=8, head_dim=128, layers=4):
    """The decode-step cache attention kernel at the full decoder's shape on this rank's share of
    the heads (fp16, one layer of a `layers`-deep cache in the reference's layouts 0 and 3):
    time by graph replay, algorithmic bytes = every cached key and value of the layer read once,
    parity of a few sequences against fp32 torch math on the same device."""
    import ppl.pmx_b200.torch_function as OPMX
    world, dev = ctx.world, ctx.device
    if heads % world or kv_heads % world:
        return None
    Hq, Hkv = heads // world, kv_heads // world
    g = torch.Generator(device=dev).manual_seed(3)
    cap = cached + 8
    rows = batch * cap
    q = torch.randn(batch, Hq, head_dim, generator=g, device=dev, dtype=torch.float16)
    kn = torch.randn(batch, Hkv, head_dim, generator=g, device=dev, dtype=torch.float16)
    vn = torch.randn(batch, Hkv, head_dim, generator=g, device=dev, dtype=torch.float16)
    start_pos = torch.full((batch,), cached, dtype=torch.int64, device=dev)
    cachestarts = torch.arange(0, rows, cap, dtype=torch.int64, device=dev)
    seqstarts = torch.arange(0, batch + 1, dtype=torch.int64, device=dev)
    kvstarts = torch.arange(0, (batch + 1) * (cached + 1), cached + 1, dtype=torch.int64, device=dev)
    one, nb, kvmax = torch.tensor([1]), torch.tensor([batch]), torch.tensor([cached + 1])
    out = {}
    for layout in (0, 3):
        shape = (rows, layers, 2, Hkv, head_dim) if layout == 0 else (layers, 2, Hkv, rows, head_dim)
        cache = torch.randn(shape, generator=g, device=dev, dtype=torch.float16)

        def call():
            return OPMX.dynamic_batching.multi_head_cache_attention(
                q, kn, vn, seqstarts, kvstarts, cachestarts, start_pos, nb, one, kvmax, cache, None, None, Hq,
                head_dim, True, False, Hkv, layers, 1, 0, 8, 0, layout)
        with torch.no_grad():
            res = call()
            graph, _ = capture(call)
            ms = timed(ctx, graph.replay, steps) / steps
            graph.reset()
        # parity on three sequences: fp32 softmax(q K^T / sqrt(d)) V over the cached rows + the new token
        view = cache[:, 1] if layout == 0 else cache[1].permute(2, 0, 1, 3)      # [rows, 2, Hkv, d]
        worst = 0.0
        for b in (0, batch // 2, batch - 1):
            r0 = int(cachestarts[b])
            keys = view[r0:r0 + cached + 1, 0].float()
            vals = view[r0:r0 + cached + 1, 1].float()
            for h in range(Hq):
                sc = keys[:, h // (Hq // Hkv)] @ q[b, h].float() / head_dim ** 0.5
                want = torch.softmax(sc, 0) @ vals[:, h // (Hq // Hkv)]
                worst = max(worst, float((res[b, h].float() - want).abs().max()))
        nbytes = 2.0 * batch * (cached + 1) * Hkv * head_dim * 2
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[f"layout{layout}"] = {"ms": ms, "algorithmic_bytes": nbytes, "achieved_gbs": gbs,
                                  "frac_of_hbm_peak": gbs / ctx.peaks["hbm_gbs"], "max_abs_err": worst,
                                  "ok": worst <= ATOL}
        del cache
    out["config"] = {"batch": batch, "cached_tokens": cached, "num_heads": Hq, "num_kv_heads": Hkv, "head_dim": head_dim,
                     "parallelism": f"tp{world}", "dtype": "f16"}
    return out


def parse_plan(text):
    from ppl.pmx_b200._cabi import GemmPlan
    if not text:
        return None
    return GemmPlan(**{k: int(v) for k, v in (item.split("=") for item in text.split(","))})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=HEADLINE, help="the workload of the headline figures")
    ap.add_argument("--extra", default=None,
                    help="comma-separated workloads reported in the `workloads` array ('none' for none; default: all "
                         "the other configurations when the headline is the default one)")
    ap.add_argument("--regions", type=int, default=5, help="timed regions of K steps per workload (median reported)")
    ap.add_argument("--no-graph", action="store_true", help="launch the step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-pdl", action="store_true", help="ordinary launches instead of programmatic dependent launch")
    ap.add_argument("--allreduce", default="auto", choices=["auto", "peer", "nccl"],
                    help="N > 1: fused combine + all-reduce kernel over NVLink peer memory, or moe_reduce + NCCL "
                         "(auto: peer when the [T,H] result is at most 4 MB)")
    ap.add_argument("--peer-algo", default="auto", choices=["auto", "push", "pull"])
    ap.add_argument("--no-dense-decode", action="store_true",
                    help="decode-size batches: gather the routed rows first instead of the gate/up projection that "
                         "reads the un-permuted tokens and overlaps the router")
    ap.add_argument("--l2-prefetch", type=int, default=None,
                    help="k-blocks of weight tiles the weight-streaming GEMMs request into L2 in front of their "
                         "shared-memory ring (library default 0 = none)")
    ap.add_argument("--attention-kernel", default="mma", choices=["mma", "simt"],
                    help="decode attention: tensor-core kernel or CUDA-core kernel")
    ap.add_argument("--stamps", action="store_true",
                    help="headline step: record %%globaltimer stamps inside the router and expert GEMM kernels of one "
                         "graph replay and print the timeline under layer.stamps")
    ap.add_argument("--token-microbatches", type=int, default=1,
                    help="N > 1, results too large for the peer kernel: runs of tokens whose all-reduce overlaps "
                         "the next run's kernels")
    ap.add_argument("--stamps-raw", action="store_true", help="with --stamps: also the per-CTA values")
    ap.add_argument("--weight-prefetch", action="store_true",
                    help="routed decode GEMMs: request the first item's weight tiles ahead of the dependency wait "
                         "(off by default: measured slower)")
    ap.add_argument("--mlp-rows", type=int, default=None,
                    help="one-launch expert kernel: gate (= up) rows per work item of the first projection (64..128)")
    ap.add_argument("--one-launch-max-tiles", type=int, default=None,
                    help="largest number of 128-row gate/up tiles (all experts) for which decode batches run both "
                         "expert projections in one launch (library default 256: the 1/4 shard)")
    ap.add_argument("--one-launch-max-unused", type=float, default=None,
                    help="one launch for both expert projections only while the chance of an expert without tokens, "
                         "((E-k)/E)^T, is below this (library default 0.15)")
    ap.add_argument("--one-launch-max-tokens", type=int, default=None,
                    help="largest decode batch that runs both expert projections in one launch (library default 128 = "
                         "the kernel's limit)")
    ap.add_argument("--no-one-launch", action="store_true",
                    help="decode-size batches on thin shards: gate/up and down projection as two launches")
    ap.add_argument("--overlap-chunks", type=int, default=1,
                    help="N > 1, results too large for the peer kernel: hidden-column slices of the down projection "
                         "whose all-reduces overlap the next slice's GEMM (1: one GEMM, one all-reduce)")
    ap.add_argument("--gemm-plan", default="", help="pmx_gemm_plan fields for the gate_up / down STAGE timings, "
                                                    "e.g. balance=2,cta_cap=128 (the step itself uses the default plan)")
    ap.add_argument("--decoder", default="auto", choices=["auto", "on", "off"],
                    help="also run one decode step of the full Mixtral-8x7B-architecture decoder (the reference model "
                         "from oracle/_ref with this package's operators swapped in); auto: when N = 8")
    ap.add_argument("--decoder-scale", type=int, default=1, help="divide the decoder's widths by this (tests)")
    ap.add_argument("--decoder-layers", type=int, default=32)
    ap.add_argument("--decoder-batch", type=int, default=64)
    ap.add_argument("--decoder-cached", type=int, default=2048)
    ap.add_argument("--attention-only", action="store_true",
                    help="measure only the decode-step cache attention kernel and print its record")
    ap.add_argument("--ffn-div", type=int, default=1,
                    help="divide the ffn size by this (small cases for profiler captures; traffic and flops scale with it)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    from ppl.pmx_b200 import workloads as W

    def shape_of(name):
        sh = W.WORKLOADS[name]
        if args.ffn_div != 1:
            sh = W.scaled(sh, I=sh.I // args.ffn_div, name=f"{sh.name}_ffn_div{args.ffn_div}")
        return sh

    shape = shape_of(args.workload)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, shape, rank)
        return

    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with "
                         f"python -m torch.distributed.run --nproc-per-node {args.gpus} bench.py --gpus {args.gpus}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    ctx = Ctx()
    ctx.args, ctx.world, ctx.rank, ctx.local_rank = args, world, rank, local_rank
    ctx.device = torch.device("cuda", local_rank)
    ctx.group, ctx.blocks, ctx.peer_failed, ctx.peaks = None, {}, False, load_peaks()
    if world > 1:
        dist.init_process_group("nccl", device_id=ctx.device)
        ctx.group = dist.new_group(list(range(world)))
    from ppl.pmx_b200 import _cabi
    if args.no_pdl:
        _cabi.lib.pmx_moe_set_programmatic_launch(0)
    if args.weight_prefetch:
        _cabi.lib.pmx_moe_set_weight_prefetch(1)
    if args.mlp_rows is not None:
        _cabi.lib.pmx_moe_dense_mlp_set_rows(args.mlp_rows)
    if args.one_launch_max_tiles is not None:
        import ppl.pmx_b200.torch_function.moe as moe_mod
        moe_mod.ONE_LAUNCH_MAX_TILES = args.one_launch_max_tiles
    if args.one_launch_max_unused is not None:
        import ppl.pmx_b200.torch_function.moe as moe_mod
        moe_mod.ONE_LAUNCH_MAX_UNUSED = args.one_launch_max_unused
    if args.one_launch_max_tokens is not None:
        import ppl.pmx_b200.torch_function.moe as moe_mod
        moe_mod.ONE_LAUNCH_MAX_TOKENS = args.one_launch_max_tokens
    if args.l2_prefetch is not None:
        _cabi.lib.pmx_moe_set_l2_prefetch(args.l2_prefetch)
    _cabi.lib.pmx_decode_cache_attention_set_kernel(["mma", "simt"].index(args.attention_kernel))
    ctx.gemm_plan = parse_plan(args.gemm_plan)

    if args.attention_only:
        rec = measure_attention(ctx, min(args.steps, 100))
        if rank == 0:
            print(json.dumps({"decode_attention": rec}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    head = measure(ctx, shape, args.steps, args.warmup, args.regions, headline=True)
    extra_names = (EXTRA_WORKLOADS if args.workload == HEADLINE else []) if args.extra is None else \
        [n for n in args.extra.split(",") if n and n != "none"]
    extras = []
    for name in extra_names:
        sh = shape_of(name)
        # fewer steps for the long steps (prefill: ~4.5 ms each), at least 10
        k_steps = max(10, min(args.steps, int(200 / max(1.0, 0.002 * sh.T))))
        try:
            rec = measure(ctx, sh, k_steps, max(3, min(args.warmup, 5)), args.regions, headline=False)
        except Exception as exc:                      # noqa: BLE001
            rec = {"workload": sh.name, "error": f"{type(exc).__name__}: {exc}"}
            if world > 1:
                raise
        if rank == 0:
            extras.append(rec)

    attention = measure_attention(ctx, min(args.steps, 100)) if args.workload == HEADLINE and args.ffn_div == 1 else None
    decoder = None
    import oracle
    want_decoder = args.decoder == "on" or (args.decoder == "auto" and world == 8 and args.workload == HEADLINE)
    if want_decoder and oracle.ref_path() is None:
        decoder = {"unavailable": "the OPMX reference is not staged under oracle/_ref (python oracle/make_ref.py)"}
    elif want_decoder:
        ctx.blocks.clear()
        torch.cuda.empty_cache()
        sc = args.decoder_scale
        cfg = dict(DECODER_FULL, num_layers=args.decoder_layers)
        if sc > 1:
            cfg.update(hidden_dim=cfg["hidden_dim"] // sc, intermediate_dim=cfg["intermediate_dim"] // sc,
                       vocab_size=cfg["vocab_size"] // sc)
        decoder = run_decoder(ctx, cfg, args.decoder_batch, args.decoder_cached, steps=3)

    if rank == 0:
        ms_step = head["ms_per_step"]
        line = {
            "metric": METRIC, "value": head["tokens_per_s"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": shape.dtype, "data": "synthetic",
            "config": head["config"],
            "repeats": head["repeats"],
            "e2e": {"value": shape.T / (head["e2e_ms_total"] / args.steps * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": head["h2d"], "d2h_bytes_per_step": head["d2h"]},
            "gpu_launches": head["gpu_launches_per_step"] * args.steps,
            "programmatic_dependent_launch": not args.no_pdl,
            "l2_prefetch_kblocks": args.l2_prefetch if args.l2_prefetch is not None else "library default",
            "clocks": head["clocks"],
            "roofline": head["roofline"],
            "roofline_down": head["roofline_down"],
            "roofline_gate_up_as_its_own_launch": head.get("roofline_gate_up_as_its_own_launch"),
            "layer": head["layer"],
            "parity": head["parity"],
            "workloads": extras,
        }
        if attention is not None:
            line["decode_attention"] = attention
        if decoder is not None:
            line["decoder"] = decoder
        if world == 1 and not args.no_cpu_baseline:
            blk = get_block(ctx, shape, full=False)
            x_host, w_router, _, _ = W.make_activations(shape, detie=False)
            wu_c, w2_c = blk.wu.weight.detach().cpu(), blk.w2.weight.detach().cpu()
            arm = CpuArm(shape)
            tokens = min(shape.T, 1024)
            times = arm.time(x_host, w_router, wu_c, w2_c, tokens, 20, 1, budget_s=15.0)
            line["cpu_baseline"] = {"value": tokens * len(times) / sum(times), "unit": UNIT, "cores": arm.cores,
                                    "kind": arm.kind, "sample": arm.describe(tokens, len(times))}
        print(json.dumps(line), flush=True)
    # Tear-down.  A CUDA graph that captured NCCL kernels must be gone before the
    # communicator is destroyed; a watchdog ends the process with an error if the
    # tear-down itself stalls (the result line is already out).
    sys.stdout.flush()
    if world > 1:
        def stalled():
            sys.stderr.write("[bench] tear-down of the process group stalled for 60 s; exiting with status 3\n")
            sys.stderr.flush()
            os._exit(3)
        watchdog = threading.Timer(60.0, stalled)
        watchdog.daemon = True
        watchdog.start()
        sync_all(ctx)
        ctx.blocks.clear()
        torch.cuda.synchronize()
        dist.destroy_process_group()
        watchdog.cancel()


if __name__ == "__main__":
    main()
