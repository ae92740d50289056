"""Tensor-parallel MoE block on 2 GPUs (NCCL) against the single-process oracle.
Skipped where fewer than two devices are visible."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        group = dist.new_group(list(range(world)))
        from oracle import moe_oracle as orc
        from ppl.pmx_b200 import workloads as W
        from ppl.pmx_b200.moe_layers import MoeFeedForward
        for base, kw in (("decode_t64", dict(H=512, I=1024)), ("prefill", dict(T=1024, H=256, I=512))):
            sh = W.scaled(W.WORKLOADS[base], **kw)
            x, wr, sc, _ = W.make_activations(sh)
            full_u, full_d = W.make_expert_weights(sh, dev)
            f = lambda t: t.detach().float().cpu().numpy()
            ref = orc.moe_block(f(x), f(wr), f(full_u), f(full_d), sh.E, sh.k, sh.dtype, scores=f(sc),
                                round_intermediates=False)
            import ppl.pmx_b200.moe_layers as layers_mod
            for fused, peer in ((True, 0), (False, 0), (True, sh.T), ("sliced", 0), ("runs", 0)):
                # "sliced": down projection + combine + all-reduce per slice of the hidden columns,
                # the all-reduce of a slice overlapping the GEMM of the next one; "runs": the
                # block per run of tokens, a run's all-reduce overlapping the next run's kernels
                layers_mod.OVERLAP_MIN_BYTES = 0 if fused in ("sliced", "runs") else 1 << 60
                blk = MoeFeedForward(sh.H, sh.I, sh.E, sh.k, group, False, fused=bool(fused),
                                     peer_reduce_tokens=peer, overlap_chunks=2 if fused == "sliced" else 1,
                                     token_microbatches=2 if fused == "runs" else 1
                                     ).to(dev, W.TORCH_DTYPE[sh.dtype])
                u, d = W.make_expert_weights(sh, dev, tp_rank=rank, tp_size=world)
                xd, scd = x.to(dev), sc.to(dev)
                with torch.no_grad():
                    blk.wu.weight.copy_(u)
                    blk.w2.weight.copy_(d)
                    for _ in range(3 if peer else 1):       # consecutive calls alternate the exchange buffers
                        out = blk(xd, router_logits=scd)
                torch.cuda.synchronize()
                np.testing.assert_allclose(f(out), ref["out"], atol=2e-2, rtol=1e-2,
                                           err_msg=f"{sh.name} fused={fused} peer={peer} rank={rank}")
                if peer:
                    blk._peer.check()
                    # the same step captured in a CUDA graph and replayed
                    side = torch.cuda.Stream()
                    side.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(side), torch.no_grad():
                        blk(xd, router_logits=scd)
                    torch.cuda.current_stream().wait_stream(side)
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph), torch.no_grad():
                        gout = blk(xd, router_logits=scd)
                    for _ in range(4):
                        graph.replay()
                    torch.cuda.synchronize()
                    np.testing.assert_allclose(f(gout), ref["out"], atol=2e-2, rtol=1e-2,
                                               err_msg=f"{sh.name} graph replay rank={rank}")
                    blk._peer.check()
                    graph.reset()
                    del graph
        q.put((rank, "ok"))
    except Exception:                            # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def _op_level(rank, world, port, q):
    """The operator-level collectives on real GPUs: moe_column_parallel_linear with
    gather_output=True (all-gather + rank-major concatenation, MoeColumnParallelLinear.py:71-78),
    moe_row_parallel_linear (all-reduce of the expanded rows, MoeRowParallelLinear.py:57-58), and
    the dense column / row parallel linears (ColumnParallelLinear.py:44-52, RowParallelLinear.py:41-45)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        group = dist.new_group(list(range(world)))
        import ppl.pmx_b200.torch_function as F
        from oracle import moe_oracle as orc
        g = torch.Generator().manual_seed(7)
        E, k, T, H, N = 4, 2, 96, 128, 256
        x = torch.randn(T, H, generator=g).half()
        sc = torch.randn(T, E, generator=g).half()
        w_col = (torch.randn(E, N, H, generator=g) / H ** 0.5).half()          # full [E, N, H]
        b_col = torch.randn(E, N, generator=g).half()
        w_row = (torch.randn(E, H, N, generator=g) / N ** 0.5).half()          # full [E, H, N]
        f = lambda t: t.float().numpy()
        xe, ew, inv, off = F.moe_select(x.to(dev), sc.to(dev), E, k)
        Nl = N // world
        shard = slice(rank * Nl, (rank + 1) * Nl)
        y = F.moe_column_parallel_linear(xe, off, w_col[:, shard].contiguous().to(dev), b_col[:, shard].contiguous().to(dev),
                                         group, E, H, N, True)
        oxe, _, _, ooff = orc.moe_select(f(x), f(sc), E, k, "f16")
        want = orc.moe_grouped_linear(oxe, ooff, f(w_col), f(b_col))
        assert y.shape == (T, k, N)
        np.testing.assert_allclose(y.float().cpu().numpy().reshape(T * k, N), want, atol=2e-2, rtol=1e-2)
        z = F.moe_row_parallel_linear(y[..., shard].contiguous(), off, w_row[:, :, shard].contiguous().to(dev), None,
                                      group, E, N, H, True)
        want_z = orc.moe_grouped_linear(orc.round_to_dtype(want, "f16"), ooff, f(w_row), None)
        np.testing.assert_allclose(z.float().cpu().numpy().reshape(T * k, H), want_z, atol=3e-2, rtol=2e-2)
        # dense linears
        wd = (torch.randn(N, H, generator=g) / H ** 0.5).half()
        bd = torch.randn(N, generator=g).half()
        yc = F.column_parallel_linear(x.to(dev), wd[shard].contiguous().to(dev), bd[shard].contiguous().to(dev), group, H, N, True)
        np.testing.assert_allclose(yc.float().cpu().numpy(), orc.linear(f(x), f(wd), f(bd)), atol=2e-2, rtol=1e-2)
        wr = (torch.randn(H, N, generator=g) / N ** 0.5).half()
        br = torch.randn(H, generator=g).half()
        yr = F.row_parallel_linear(yc[:, shard].contiguous(), wr[:, shard].contiguous().to(dev), br.to(dev), group, N, H, True)
        np.testing.assert_allclose(yr.float().cpu().numpy(), orc.linear(orc.round_to_dtype(orc.linear(f(x), f(wd), f(bd)), "f16"),
                                                                        f(wr), f(br)), atol=3e-2, rtol=2e-2)
        q.put((rank, "ok"))
    except Exception:                            # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def _spawn(target, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


def test_operator_level_collectives_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _spawn(_op_level)


def _alternating(rank, world, port, q):
    """One set of exchange buffers, token counts that change from call to call (64, 8, 64,
    8, ...) and one rank held back on the host between calls: a fast rank starts the next
    exchange while the slow one may still be reading the previous one."""
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        group = dist.new_group(list(range(world)))
        import ppl.pmx_b200.torch_function as F
        from ppl.pmx_b200.peer_reduce import PeerCombine
        N, k = 1024, 2
        for algo in ("push", "pull"):
            peer = PeerCombine(group, 64, N, torch.float16, dev, algorithm=algo)
            for call, T in enumerate([64, 8, 64, 8, 1, 64, 33, 8]):
                g = torch.Generator().manual_seed(call)
                w = torch.rand(T, k, generator=g).half().to(dev)
                inv = torch.randperm(T * k, generator=g).view(T, k).to(dev)
                ys = [torch.randn(T * k, N, generator=g).half() for _ in range(world)]
                if rank == 1:
                    time.sleep(0.02)              # the slow rank
                out = peer.combine_allreduce(ys[rank].to(dev), w, inv, k)
                want = sum(F.moe_reduce(y.to(dev).view(T, k, N), w, inv, k).float() for y in ys)
                torch.testing.assert_close(out.float(), want, atol=2e-2, rtol=1e-2,
                                           msg=f"{algo} call {call} T={T} rank {rank}")
            peer.check()
        q.put((rank, "ok"))
    except Exception:                            # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def test_exchange_buffers_survive_changing_token_counts_and_a_slow_rank():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_alternating, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


def test_tensor_parallel_block_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"
