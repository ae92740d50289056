"""Tensor-parallel host logic on CPU: world_size-2 (and 4) gloo ranks run the
MoE block modules with the CUDA calls replaced, in this test only, by the numpy
oracle.  What is under test is everything around the kernels: weight sharding,
which rank adds the bias, the all-reduce placement of the operator API
(expanded rows, as the reference) and of the fused block (after the combine),
and the all-gather of the column-parallel output."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _install_cpu_stand_ins():
    """Route the library calls to the oracle (tests only)."""
    from oracle import moe_oracle as orc
    import ppl.pmx_b200.torch_function.moe as moe
    import ppl.pmx_b200.torch_function as F
    import ppl.pmx_b200.moe_layers as layers

    def t(a):
        return torch.from_numpy(np.ascontiguousarray(a))

    def grouped(X, off, W, B=None, *, swiglu=False, beta=1.0, zero_outside=True, plan=None, return_workspace=False):
        y = orc.moe_grouped_linear(X.reshape(-1, X.shape[-1]).numpy(), off.numpy(), W.detach().numpy(),
                                   None if B is None else B.detach().numpy())
        if swiglu:
            y = orc.swiglu(y, beta)
        y = t(y).view(*X.shape[:-1], -1)
        return (y, None) if return_workspace else y

    def select(X, scores, E, k):
        xe, ew, inv, off = orc.moe_select(X.reshape(-1, X.shape[-1]).numpy(), scores.reshape(-1, E).numpy(), E, k)
        return t(xe).view(*X.shape[:-1], k, -1), t(ew).view(*X.shape[:-1], k), t(inv).view(*X.shape[:-1], k), t(off)

    def reduce(Y, w, inv, k):
        return t(orc.moe_reduce(Y.reshape(-1, Y.shape[-1]).numpy(), w.numpy(), inv.numpy(), k)).view(*w.shape[:-1], -1)

    moe.moe_grouped_linear = grouped
    layers.moe_grouped_linear = grouped
    F.moe_select = select
    F.moe_reduce = reduce
    F.swiglu = lambda X, beta=1.0: t(orc.swiglu(X.numpy(), beta))


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        group = dist.new_group(list(range(world)), backend="gloo")
        _install_cpu_stand_ins()
        from oracle import moe_oracle as orc
        from ppl.pmx_b200 import workloads as W
        from ppl.pmx_b200.moe_layers import MoeFeedForward, MoeColumnParallelLinear
        sh = W.scaled(W.WORKLOADS["small_f32"], T=40, H=32, I=64)
        x, wr, sc, _ = W.make_activations(sh)
        full_u, full_d = W.make_expert_weights(sh, "cpu")
        ref = orc.moe_block(x.numpy(), wr.numpy(), full_u.numpy(), full_d.numpy(), sh.E, sh.k, "f32",
                            scores=sc.numpy())
        g = torch.Generator().manual_seed(5)
        bias_u_full = torch.randn(sh.E, 2 * sh.I, generator=g)
        bias_d = torch.randn(sh.E, sh.H, generator=g)
        Il = sh.I // world
        bias_u = torch.cat([bias_u_full[:, rank * Il:(rank + 1) * Il],
                            bias_u_full[:, sh.I + rank * Il: sh.I + (rank + 1) * Il]], 1)
        ref_b = None
        import ppl.pmx_b200.moe_layers as layers_mod
        for fused in (True, False, "sliced", "runs"):
            # "sliced": the fused block with the down projection, combine and all-reduce done
            # per slice of the hidden columns (the all-reduces overlap the next slice's GEMM);
            # "runs": the block per run of tokens, a run's all-reduce overlapping the next run
            layers_mod.OVERLAP_MIN_BYTES = 0 if fused in ("sliced", "runs") else 1 << 60
            for with_bias in (False, True):
                blk = MoeFeedForward(sh.H, sh.I, sh.E, sh.k, group, with_bias, fused=bool(fused),
                                     overlap_chunks=2 if fused == "sliced" else 1,
                                     token_microbatches=2 if fused == "runs" else 1)
                u, d = W.make_expert_weights(sh, "cpu", tp_rank=rank, tp_size=world)
                assert blk.wu.weight.shape == u.shape and blk.w2.weight.shape == d.shape
                with torch.no_grad():
                    blk.wu.weight.copy_(u)
                    blk.w2.weight.copy_(d)
                    if with_bias:
                        blk.wu.bias.copy_(bias_u)
                        blk.w2.bias.copy_(bias_d)
                    out = blk(x, router_logits=sc)
                if with_bias:
                    if ref_b is None:
                        xe, ew, inv, off = orc.moe_select(x.numpy(), sc.numpy(), sh.E, sh.k)
                        h = orc.swiglu(orc.moe_grouped_linear(xe, off, full_u.numpy(), bias_u_full.numpy()))
                        y = orc.moe_grouped_linear(h, off, full_d.numpy(), bias_d.numpy())
                        ref_b = orc.moe_reduce(y, ew, inv, sh.k)
                    want = ref_b
                else:
                    want = ref["out"]
                np.testing.assert_allclose(out.numpy(), want, atol=2e-5, rtol=1e-4,
                                           err_msg=f"fused={fused} bias={with_bias} rank={rank}")
        # gather_output=True: rank-major concatenation of the N shards (MoeColumnParallelLinear.py:71-78)
        col = MoeColumnParallelLinear(group, sh.E, sh.H, 2 * sh.I, bias_term=False, gather_output=True)
        u, _ = W.make_expert_weights(sh, "cpu", tp_rank=rank, tp_size=world)
        with torch.no_grad():
            col.weight.copy_(u)
        xe, ew, inv, off = orc.moe_select(x.numpy(), sc.numpy(), sh.E, sh.k)
        with torch.no_grad():
            y = col(torch.from_numpy(xe), torch.from_numpy(off))
        assert y.shape == (sh.T * sh.k, 2 * sh.I)
        mine = orc.moe_grouped_linear(xe, off, u.numpy())
        np.testing.assert_allclose(y[:, rank * 2 * Il:(rank + 1) * 2 * Il].numpy(), mine, atol=1e-5)
        q.put((rank, "ok"))
    except Exception as e:                       # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def _leaver(rank, world, port, q):
    """Failure detection on the host side: the ranks run two steps together, then the last
    rank leaves between steps (no collective of its own in flight).  The others notice in
    their next collective, which ends with an error after the group's short timeout
    instead of blocking forever."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        group = dist.new_group(list(range(world)), backend="gloo", timeout=datetime.timedelta(seconds=5))
        _install_cpu_stand_ins()
        from ppl.pmx_b200 import workloads as W
        from ppl.pmx_b200.moe_layers import MoeFeedForward
        sh = W.scaled(W.WORKLOADS["small_f32"], T=16, H=32, I=96)
        x, _, sc, _ = W.make_activations(sh)
        blk = MoeFeedForward(sh.H, sh.I, sh.E, sh.k, group, False)
        u, d = W.make_expert_weights(sh, "cpu", tp_rank=rank, tp_size=world)
        with torch.no_grad():
            blk.wu.weight.copy_(u)
            blk.w2.weight.copy_(d)
            for _ in range(2):
                blk(x, router_logits=sc)            # steps with everybody present
            if rank == world - 1:
                q.put((rank, "left"))
                return                                # leaves between steps
            try:
                blk(x, router_logits=sc)            # the all-reduce of this step cannot complete
                q.put((rank, "no error"))
            except Exception as exc:                  # noqa: BLE001
                q.put((rank, f"error: {type(exc).__name__}"))
    except Exception:                                 # noqa: BLE001
        import traceback
        q.put((rank, traceback.format_exc()))
    finally:
        if rank == world - 1:
            q.close()
            q.join_thread()                           # the message is out before the process dies
            os._exit(0)                               # gone without a clean shutdown, like a crashed rank
        try:
            dist.destroy_process_group()
        except Exception:                             # noqa: BLE001
            pass


def test_a_rank_that_leaves_between_steps_is_detected_on_gloo():
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_leaver, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert results[world - 1] == "left"
    for r in range(world - 1):
        assert results[r].startswith("error"), f"rank {r} did not notice the missing rank: {results[r]}"


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_block_on_gloo(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"
