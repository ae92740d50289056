#!/usr/bin/env python
"""MoE-layer throughput of the B200 implementation (and of the CPU reference arm).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode_t64] [--impl reference]

One "step" is one call of the Mixtral MoE block (router gate -> moe_select ->
gate/up projection + SwiGLU -> down projection -> moe_reduce -> all-reduce when
N > 1) on one batch of seeded synthetic tokens.  With N > 1 (launched by
torchrun, one rank per GPU) every expert's intermediate dimension is sharded
over the ranks, so the total work is fixed as N grows ("strong" scaling).

The line printed by rank 0:
  value     tokens/s with the inputs resident in HBM, K replays of the captured
            CUDA graph of the step, CUDA events on the launching stream, max over ranks
  e2e       the same with the step's input copied from pinned host memory and
            its output copied back inside the timed region, every step
  roofline  the dominant kernel (gate/up grouped GEMM): its launch alone captured in a
            CUDA graph and replayed K times between two CUDA events, in the same run
  cpu_baseline  the CPU port of the reference algorithm (oracle/cpu_port.py) on
            the host cores of this machine, a bounded sample of the same workload
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


# ------------------------------------------------------------------------------ CPU arm
def cpu_pass(shape, x, w_router, wu, w2, tokens):
    from oracle import cpu_port
    out, _ = cpu_port.moe_block(x[:tokens], w_router, wu, w2, shape.E, shape.k)
    return out


def time_cpu(shape, x, w_router, wu, w2, tokens, steps, warmup, budget_s=None):
    torch.set_num_threads(os.cpu_count() or 1)
    with torch.inference_mode():
        for _ in range(warmup):
            cpu_pass(shape, x, w_router, wu, w2, tokens)
        times = []
        t_begin = time.perf_counter()
        for _ in range(steps):
            t0 = time.perf_counter()
            cpu_pass(shape, x, w_router, wu, w2, tokens)
            times.append(time.perf_counter() - t0)
            if budget_s is not None and time.perf_counter() - t_begin > budget_s:
                break
    return times


def run_reference(args, shape, rank):
    """The reference's CPU torch path for the same workload, on this machine's host cores."""
    if rank != 0:
        return
    from ppl.pmx_b200 import workloads as W
    x, w_router, scores, _ = W.make_activations(shape, detie=False)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    wu, w2 = W.make_expert_weights(shape, dev)
    wu, w2 = wu.cpu(), w2.cpu()
    tokens = min(shape.T, 1024)
    times = time_cpu(shape, x, w_router, wu, w2, tokens, args.steps, min(args.warmup, 2))
    total = sum(times)
    value = tokens * len(times) / total
    sample = f"first {tokens} of {shape.T} tokens per step, all {shape.E} experts' full weights, {len(times)} steps"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": len(times), "warmup": min(args.warmup, 2), "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": shape.dtype,
        "data": "synthetic", "config": workload_config(shape, 1, "cpu"),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(shape, tp, where):
    return {"workload": shape.name, "tokens": shape.T, "hidden": shape.H, "experts": shape.E,
            "experts_per_token": shape.k, "ffn": shape.I, "parallelism": f"tp{tp}",
            "l2": "weights per rank exceed the 126 MB L2, no flush between steps", "device": where}


# ------------------------------------------------------------------------------ GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_t64")
    ap.add_argument("--no-graph", action="store_true", help="launch the step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--allreduce", default="auto", choices=["auto", "peer", "nccl"],
                    help="N > 1: fused combine + all-reduce kernel over NVLink peer memory, or moe_reduce + NCCL "
                         "(auto: peer when the [T,H] result is at most 4 MB)")
    ap.add_argument("--ffn-div", type=int, default=1,
                    help="divide the ffn size by this (small cases for profiler captures; traffic and flops scale with it)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    from ppl.pmx_b200 import workloads as W
    shape = W.WORKLOADS[args.workload]
    if args.ffn_div != 1:
        shape = W.scaled(shape, I=shape.I // args.ffn_div, name=f"{shape.name}_ffn_div{args.ffn_div}")
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
    device = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        group = dist.new_group(list(range(world)))

    import ppl.pmx_b200.torch_function as OPMX
    from ppl.pmx_b200 import _cabi
    from ppl.pmx_b200.moe_layers import MoeFeedForward
    from ppl.pmx_b200.torch_function.moe import moe_grouped_linear

    dt = W.TORCH_DTYPE[shape.dtype]
    x_host, w_router, _, _ = W.make_activations(shape, detie=False)
    x_host = x_host.pin_memory()
    out_host = torch.empty(shape.T, shape.H, dtype=dt).pin_memory()
    result_bytes = shape.T * shape.H * torch.empty((), dtype=dt).element_size()
    use_peer = world > 1 and (args.allreduce == "peer" or (args.allreduce == "auto" and result_bytes <= (4 << 20)))
    blk = MoeFeedForward(shape.H, shape.I, shape.E, shape.k, group, False,
                         peer_reduce_tokens=shape.T if use_peer else 0).to(device, dt)
    wu, w2 = W.make_expert_weights(shape, device, tp_rank=rank, tp_size=world)
    with torch.no_grad():
        blk.gate.weight.copy_(w_router)
        blk.wu.weight.copy_(wu)
        blk.w2.weight.copy_(w2)
    del wu, w2
    x_dev = x_host.to(device)
    E, k = shape.E, shape.k

    def step():
        with torch.no_grad():
            return blk(x_dev)

    if use_peer:
        # the peer-memory exchange needs the ranks' buffers mapped into each other
        # (symmetric memory); if this machine refuses, say so and use NCCL
        try:
            step()
            torch.cuda.synchronize()
            ok = torch.ones(1, device=device)
        except Exception as exc:                      # noqa: BLE001
            print(f"[bench] rank {rank}: peer-memory all-reduce unavailable ({exc}); using NCCL", file=sys.stderr)
            ok = torch.zeros(1, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if ok.item() == 0:
            use_peer = False
            blk.peer_reduce_tokens = 0
            blk._peer = None

    def sync_all():
        if world > 1:
            dist.barrier(group=group)
        torch.cuda.synchronize()

    # warm-up (eager), then capture one step
    for _ in range(args.warmup):
        out = step()
    torch.cuda.synchronize()
    launches_before = _cabi.lib.pmx_moe_kernel_launches()
    out = step()
    torch.cuda.synchronize()
    launches_per_step = _cabi.lib.pmx_moe_kernel_launches() - launches_before
    graph = None
    if not args.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            out = step()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = step()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()

    def run_step():
        if graph is not None:
            graph.replay()
            return out
        return step()

    def timed(fn, steps):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync_all()
        ms = torch.tensor([e0.elapsed_time(e1)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=group)
        return float(ms.item())

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True)
        o = run_step()
        out_host.copy_(o, non_blocking=True)

    sampler = ClockSampler(physical_gpu_index(local_rank))
    with sampler:
        ms_total = timed(run_step, args.steps)
        ms_e2e = timed(e2e_step, args.steps)

        # per-stage pass: every stage of the step is captured in a CUDA graph of its own and
        # replayed K times between two CUDA events (no host launch gaps inside the figure);
        # with --no-graph the stages are launched eagerly instead
        names = ["gate", "select", "route_select", "gate_up", "down", "reduce", "allreduce", "reduce_allreduce",
                 "skip_rms_norm", "norm_route_select"]
        kernel_ms = {n: 0.0 for n in names}
        keep = []

        def stage(name, fn):
            with torch.no_grad():
                r = fn()                                   # eager: produces the next stage's inputs
                if args.no_graph:
                    run = fn
                else:
                    side = torch.cuda.Stream()
                    side.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(side):
                        fn()
                    torch.cuda.current_stream().wait_stream(side)
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        fn()
                    keep.append(g)
                    run = g.replay
                kernel_ms[name] = timed(run, args.steps) / args.steps
            return r

        sync_all()
        if OPMX.moe_route_select(x_dev, blk.gate.weight, E, k) is not None:
            _, xe, ew, inv, off = stage("route_select", lambda: OPMX.moe_route_select(x_dev, blk.gate.weight, E, k))
        else:
            logits = stage("gate", lambda: torch.nn.functional.linear(x_dev, blk.gate.weight))
            xe, ew, inv, off = stage("select", lambda: OPMX.moe_select(x_dev, logits, E, k))
        h = stage("gate_up", lambda: moe_grouped_linear(xe.view(-1, shape.H), off, blk.wu.weight, None,
                                                        swiglu=True, zero_outside=False))
        y = stage("down", lambda: moe_grouped_linear(h, off, blk.w2.weight, None, zero_outside=False))
        if use_peer:
            stage("reduce_allreduce", lambda: blk._peer.combine_allreduce(y, ew, inv, k))
        else:
            o = stage("reduce", lambda: OPMX.moe_reduce(y.view(shape.T, k, -1), ew, inv, k))
            if world > 1:
                stage("allreduce", lambda: dist.all_reduce(o, group=group))
        # the normalisation in front of the block (not part of the step): x + skip -> RMSNorm
        norm_w = torch.ones(shape.H, device=device, dtype=dt)
        skip_dev = torch.randn_like(x_dev)
        stage("skip_rms_norm", lambda: OPMX.skip_rms_norm(x_dev, norm_w, skip_dev, -1, 1e-5))
        if OPMX.moe_norm_route_select(x_dev, skip_dev, norm_w, 1e-5, blk.gate.weight, E, k) is not None:
            stage("norm_route_select",
                  lambda: OPMX.moe_norm_route_select(x_dev, skip_dev, norm_w, 1e-5, blk.gate.weight, E, k))
        sync_all()
        for g in keep:
            g.reset()
        del keep
    active = int((off[1:] - off[:-1]).gt(0).sum().item())
    # phase boundaries of the last fused combine + all-reduce call (CTA 0 of this rank), from
    # the %globaltimer stamps the kernel leaves in its control block (byte 512, 8 x u64)
    ar_phases = None
    if use_peer and getattr(blk, "_peer", None) is not None:
        try:
            import struct
            st = struct.unpack("8Q", bytes(blk._peer.buffer[512:576].cpu().tolist()))
            ar_phases = {"combine_done": st[1] - st[0], "epoch_published": st[2] - st[0],
                         "peers_seen": st[3] - st[0], "sum_done": st[4] - st[0]}
        except Exception:                                 # noqa: BLE001  (diagnostic only)
            ar_phases = None

    if rank == 0:
        peaks = load_peaks()
        work = W.algorithmic_work(shape, world, active)
        ms_step = ms_total / args.steps
        value = shape.T / (ms_step * 1e-3)
        e2e_value = shape.T / (ms_e2e / args.steps * 1e-3)
        # dominant kernel: the gate/up grouped GEMM
        t_gu = kernel_ms["gate_up"] * 1e-3
        ai = work["flops_gate_up"] / work["bytes_gate_up"]
        clocks = sampler.summary()
        # tensor peak: the burst figure when the timed region ran at (nearly) full SM clock,
        # the sustained one when the power cap had pulled the clock down
        burst = bool(clocks["sm_mhz"] and clocks["sm_max_mhz"] and clocks["sm_mhz"] >= 0.9 * clocks["sm_max_mhz"])
        tensor_peak = peaks["bf16_tflops"] if burst else peaks["bf16_tflops_sustained"]
        tensor_peak_kind = "burst" if burst else "sustained"
        ridge = tensor_peak * 1e12 / (peaks["hbm_gbs"] * 1e9)
        if ai < ridge:
            achieved = work["bytes_gate_up"] / t_gu / 1e9
            roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"]}
        else:
            achieved = work["flops_gate_up"] / t_gu / 1e12
            roof = {"bound": "tensor", "achieved": achieved, "peak": tensor_peak,
                    "unit": "TFLOP/s", "frac": achieved / tensor_peak, "peak_kind": tensor_peak_kind}
        # DRAM traffic of the launch = algorithmic bytes x the ratio ncu measured on a
        # reduced-ffn case of the same kernel (profiles/grouped_gemm_tc_*.md); traffic is
        # >99 % weights and scales with the ffn size
        ratio = TRAFFIC_RATIO.get(roof["bound"])
        roof.update({"traffic": work["bytes_gate_up"] * ratio if ratio else None, "kernel": "gate/up grouped GEMM with SwiGLU epilogue (grouped_gemm_tc_kernel; grouped_gemm_tc_pair_kernel for >= 1024 rows per expert)",
                     "kernel_ms": kernel_ms["gate_up"], "peak_source": peaks["source"],
                     "algorithmic_bytes": work["bytes_gate_up"], "algorithmic_flops": work["flops_gate_up"],
                     "timing": "CUDA events around K back-to-back replays of a CUDA graph holding this launch alone, same run"})
        # whole-layer figures against the layer's own roofline
        layer_floor_s = max(work["bytes"] / (peaks["hbm_gbs"] * 1e9), work["flops"] / (tensor_peak * 1e12))
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": shape.dtype, "data": "synthetic",
            "config": workload_config(shape, world, "B200"),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * x_host.element_size(),
                    "d2h_bytes_per_step": out_host.numel() * out_host.element_size()},
            "gpu_launches": int(launches_per_step) * args.steps,
            "clocks": clocks,
            "roofline": roof,
            "layer": {"ms_floor": layer_floor_s * 1e3, "frac_of_roofline": layer_floor_s * 1e3 / ms_step,
                      "active_experts": active, "graph": graph is not None,
                      "allreduce": ("peer-memory kernel fused with the combine" if use_peer else "nccl") if world > 1 else None,
                      "allreduce_phases_ns": ar_phases,
                      "kernel_ms": {n: round(v, 5) for n, v in kernel_ms.items()
                                    if n not in ("skip_rms_norm", "norm_route_select")},
                      "front_end": {"skip_rms_norm_ms": round(kernel_ms["skip_rms_norm"], 5),
                                    "norm_route_select_ms": round(kernel_ms["norm_route_select"], 5) or None,
                                    "gbs": 4 * x_host.numel() * x_host.element_size() / (kernel_ms["skip_rms_norm"] * 1e-3) / 1e9}},
        }
        if world == 1 and not args.no_cpu_baseline:
            wu_c, w2_c = blk.wu.weight.detach().cpu(), blk.w2.weight.detach().cpu()
            tokens = min(shape.T, 1024)
            times = time_cpu(shape, x_host, w_router, wu_c, w2_c, tokens, 20, 1, budget_s=15.0)
            line["cpu_baseline"] = {
                "value": tokens * len(times) / sum(times), "unit": UNIT, "cores": torch.get_num_threads(),
                "kind": "port",
                "sample": f"first {tokens} of {shape.T} tokens, full expert weights, {len(times)} passes after 1 warm-up"}
        print(json.dumps(line), flush=True)
    # Tear-down.  A CUDA graph that captured NCCL kernels must be gone before the
    # communicator is destroyed; a watchdog ends the process if the tear-down
    # itself stalls (the result line is already out).
    sys.stdout.flush()
    if world > 1:
        watchdog = threading.Timer(30.0, lambda: os._exit(0))
        watchdog.daemon = True
        watchdog.start()
        sync_all()
        if graph is not None:
            graph.reset()
            del graph
        torch.cuda.synchronize()
        dist.destroy_process_group()
        watchdog.cancel()


if __name__ == "__main__":
    main()
