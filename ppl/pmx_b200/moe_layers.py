"""Weight-owning modules of the MoE path and the fused Mixtral MoE block.

`MoeColumnParallelLinear` / `MoeRowParallelLinear` mirror the reference modules
(model_zoo/ModelParallel.py:127-159 and :162-196): same constructor arguments,
parameter names and tensor-parallel shapes, so a reference state dict loads
unchanged.  `MoeFeedForward` mirrors the Mixtral block
(model_zoo/mixtral/modeling/dynamic_batching/Model.py:155-214) and runs it as
  gate linear -> moe_select -> gate/up GEMM with SwiGLU in the epilogue ->
  down GEMM -> moe_reduce -> one all-reduce of [T,H] over the TP group.
The reference all-reduces the expanded [T*k,H] rows before the weighted combine
(MoeRowParallelLinear.py:57-58); combining first is the same sum in another
order and moves k times fewer bytes over NVLink.
"""
from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist
from torch import nn

from . import torch_function as OPMX
from ._cabi import GemmPlan
from .torch_function.moe import (moe_grouped_linear, moe_route_select, moe_norm_route_select, moe_dense_gate_up,
                                 dense_gate_up_covers, moe_dense_mlp, dense_mlp_covers, dense_mlp_check)

# below this many bytes of [T,H] result one all-reduce is cheaper than overlapped slices
OVERLAP_MIN_BYTES = 8 << 20


# set to True to wrap the stages of MoeFeedForward in NVTX ranges (visible in a profiler
# timeline; a few host microseconds per eager call, nothing in a replayed CUDA graph)
NVTX = False


def _range(name: str):
    return torch.cuda.nvtx.range(name) if NVTX else contextlib.nullcontext()


def _world(proc_group) -> int:
    return 1 if proc_group is None else proc_group.size()


class Linear(nn.Module):
    """weight [out_features, in_features] (ModelLayers.py:51-69)."""

    def __init__(self, in_features: int, out_features: int, bias_term: bool = True) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight = nn.Parameter(torch.ones(out_features, in_features))
        if bias_term:
            self.bias = nn.Parameter(torch.zeros(out_features))
        else:
            self.register_parameter("bias", None)

    def forward(self, X: torch.Tensor):
        return OPMX.linear(X, self.weight, self.bias, self.in_features, self.out_features)


class ColumnParallelLinear(nn.Module):
    """weight [out_features/tp, in_features] (ModelParallel.py:61-92)."""

    def __init__(self, proc_group, in_features: int, out_features: int, bias_term: bool = True,
                 gather_output: bool = True) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.gather_output = gather_output
        self.proc_group = proc_group
        world_size = _world(proc_group)
        assert out_features % world_size == 0, "{} is not divisible by {}".format(out_features, world_size)
        self.out_features_per_partition = out_features // world_size
        self.weight = nn.Parameter(torch.ones(self.out_features_per_partition, in_features))
        if bias_term:
            self.bias = nn.Parameter(torch.zeros(self.out_features_per_partition))
        else:
            self.register_parameter("bias", None)

    def forward(self, X: torch.Tensor):
        return OPMX.column_parallel_linear(X, self.weight, self.bias, self.proc_group, self.in_features,
                                           self.out_features, self.gather_output)


class RowParallelLinear(nn.Module):
    """weight [out_features, in_features/tp] (ModelParallel.py:95-124)."""

    def __init__(self, proc_group, in_features: int, out_features: int, bias_term: bool = True,
                 input_is_parallel: bool = False) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.input_is_parallel = input_is_parallel
        self.proc_group = proc_group
        world_size = _world(proc_group)
        assert in_features % world_size == 0, "{} is not divisible by {}".format(in_features, world_size)
        self.in_features_per_partition = in_features // world_size
        self.weight = nn.Parameter(torch.ones(out_features, self.in_features_per_partition))
        if bias_term:
            self.bias = nn.Parameter(torch.zeros(out_features))
        else:
            self.register_parameter("bias", None)

    def forward(self, X: torch.Tensor):
        return OPMX.row_parallel_linear(X, self.weight, self.bias, self.proc_group, self.in_features,
                                        self.out_features, self.input_is_parallel)


class MoeColumnParallelLinear(nn.Module):
    """weight [E, out_features/tp, in_features] (ModelParallel.py:147-149)."""

    def __init__(self, proc_group, num_experts: int, in_features: int, out_features: int,
                 bias_term: bool = True, gather_output: bool = True) -> None:
        super().__init__()
        self.num_experts = num_experts
        self.in_features = in_features
        self.out_features = out_features
        self.gather_output = gather_output
        self.proc_group = proc_group
        world_size = _world(proc_group)
        assert out_features % world_size == 0, "{} is not divisible by {}".format(out_features, world_size)
        self.out_features_per_partition = out_features // world_size
        self.weight = nn.Parameter(torch.ones(num_experts, self.out_features_per_partition, in_features))
        if bias_term:
            self.bias = nn.Parameter(torch.zeros(num_experts, self.out_features_per_partition))
        else:
            self.register_parameter("bias", None)

    def forward(self, X: torch.Tensor, expert_offset: torch.Tensor):
        return OPMX.moe_column_parallel_linear(X, expert_offset, self.weight, self.bias, self.proc_group,
                                               self.num_experts, self.in_features, self.out_features,
                                               self.gather_output)


class MoeRowParallelLinear(nn.Module):
    """weight [E, out_features, in_features/tp] (ModelParallel.py:182-184)."""

    def __init__(self, proc_group, num_experts: int, in_features: int, out_features: int,
                 bias_term: bool = True, input_is_parallel: bool = False) -> None:
        super().__init__()
        self.num_experts = num_experts
        self.in_features = in_features
        self.out_features = out_features
        self.input_is_parallel = input_is_parallel
        self.proc_group = proc_group
        world_size = _world(proc_group)
        assert in_features % world_size == 0, "{} is not divisible by {}".format(in_features, world_size)
        self.in_features_per_partition = in_features // world_size
        self.weight = nn.Parameter(torch.ones(num_experts, out_features, self.in_features_per_partition))
        if bias_term:
            self.bias = nn.Parameter(torch.zeros(num_experts, out_features))
        else:
            self.register_parameter("bias", None)

    def forward(self, X: torch.Tensor, expert_offset: torch.Tensor):
        return OPMX.moe_row_parallel_linear(X, expert_offset, self.weight, self.bias, self.proc_group,
                                            self.num_experts, self.in_features, self.out_features,
                                            self.input_is_parallel)


class MoeFeedForward(nn.Module):
    """The Mixtral MoE feed-forward block with the fused gate/up projection
    `wu = [w1 ; w3]` (Model.py:171-174, weight packing Model.py:399-413).

    fused=True  : SwiGLU in the GEMM epilogue, combine before the all-reduce.
    fused=False : the reference's operator sequence and collective placement,
                  one library call per operator (Model.py:191-211)."""

    def __init__(self, hidden_dim: int, intermediate_dim: int, num_experts: int,
                 num_experts_per_token: int, proc_group=None, linear_bias_term: bool = False,
                 fused: bool = True, peer_reduce_tokens: int = 0, peer_algorithm: str = "auto",
                 overlap_chunks: int = 1, dense_decode: bool = True, one_launch_experts: bool = True,
                 token_microbatches: int = 1) -> None:
        super().__init__()
        self.num_experts = num_experts
        self.num_experts_per_token = num_experts_per_token
        self.proc_group = proc_group
        self.fused = fused
        self.hidden_dim = hidden_dim
        # peer_reduce_tokens > 0: for up to that many tokens the combine and the
        # all-reduce run as one kernel over NVLink peer memory (set up on first use)
        self.peer_reduce_tokens = peer_reduce_tokens
        self.peer_algorithm = peer_algorithm
        # tensor-parallel batches too large for the peer kernel: hidden-column slices whose
        # all-reduces overlap the following slice's GEMM (1 = one GEMM, one all-reduce: the
        # default, because on B200 the slices measured SLOWER: 0.99 against 0.90 ms per prefill
        # step at 8 ranks, 2.52 against 2.42 ms at 2 -- four thinner GEMMs, four combines and a
        # concatenation cost more than the overlapped part of the all-reduce gains)
        self.overlap_chunks = overlap_chunks
        # decode-size batches: gate/up projection from the un-permuted tokens, overlapping the router
        self.dense_decode = dense_decode
        # ... and, where it is covered, both expert projections in one launch
        self.one_launch_experts = one_launch_experts
        self._mlp_ws = None
        # tensor-parallel batches too large for the peer kernel: the batch is cut into this many
        # runs of tokens; the all-reduce of one run (NCCL, on the process group's own stream)
        # overlaps the whole block of the next run.  Routing is per token, so the result is the
        # same as for the whole batch.
        self.token_microbatches = token_microbatches
        self._defer_allreduce = False
        self._pending = []
        self._peer = None
        self._last_workspaces = ()     # status words of the last step's expert GEMMs, for check()
        self.gate = Linear(hidden_dim, num_experts, bias_term=False)
        self.wu = MoeColumnParallelLinear(proc_group, num_experts, hidden_dim, 2 * intermediate_dim,
                                          bias_term=linear_bias_term, gather_output=False)
        self.w2 = MoeRowParallelLinear(proc_group, num_experts, intermediate_dim, hidden_dim,
                                       bias_term=linear_bias_term, input_is_parallel=True)

    def forward_from_residual(self, x: torch.Tensor, skip: torch.Tensor | None, norm_weight: torch.Tensor,
                              eps: float = 1e-5):
        """`ffn_norm` + the block: what TransformerBlock.forward does at Model.py:261-266.
        -> (ffn, h) with h = x + skip, the residual stream handed to the next layer.  For
        decode-size batches the norm, the router gate and the select are one launch."""
        E, k = self.num_experts, self.num_experts_per_token
        tokens = x.numel() // x.shape[-1]
        # one token per block is where the single launch pays (measured on B200: 16.2 us against
        # 4.2 + 14.1 us at 64 tokens, but 26.6 against 6.2 + 18.5 us at 256)
        fused = None
        if self.fused and tokens <= 128:
            fused = moe_norm_route_select(x, skip, norm_weight, eps, self.gate.weight, E, k)
        if fused is None:
            norm, h = OPMX.skip_rms_norm(x, norm_weight, skip, -1, eps)
            return self.forward(norm), h
        h, _, x_experts, expert_weights, invert_permutation, expert_offset = fused
        return self._experts(x_experts, expert_weights, invert_permutation, expert_offset), h

    def forward(self, x: torch.Tensor, router_logits: torch.Tensor | None = None) -> torch.Tensor:
        E, k = self.num_experts, self.num_experts_per_token
        routed = None
        tokens = x.numel() // x.shape[-1] if x.shape[-1] else 0
        n_mb = self.token_microbatches
        if (n_mb > 1 and self.fused and not self._defer_allreduce
                and _world(self.proc_group) > 1 and tokens % n_mb == 0
                and tokens // n_mb * self.hidden_dim * x.element_size() >= OVERLAP_MIN_BYTES
                and not (self.peer_reduce_tokens >= tokens and self._peer_fits(tokens, x.dtype))):
            return self._forward_microbatched(x, router_logits, n_mb)
        one_launch = (self.one_launch_experts and self.wu.bias is None and self.w2.bias is None and tokens > 0
                      and dense_mlp_covers(tokens, self.wu.weight, self.w2.weight, k))
        if (router_logits is None and self.fused and self.dense_decode and tokens > 0
                and (one_launch or dense_gate_up_covers(tokens, self.wu.weight, k))):
            # decode-size batch with (almost surely) every expert in use: the gate/up projection
            # reads the un-permuted tokens and streams its weights while the router is running
            with _range("moe.route_select"):
                routed = moe_route_select(x, self.gate.weight, E, k, gather=False)
            if routed is not None:
                _, _, expert_weights, invert_permutation, expert_offset = routed
                if one_launch:
                    with _range("moe.experts(one launch)"):
                        y, self._mlp_ws = moe_dense_mlp(x, invert_permutation, expert_offset, self.wu.weight,
                                                        self.w2.weight, return_workspace=True)
                    self._last_workspaces = ()
                    return self._combine(y, expert_weights, invert_permutation)
                with _range("moe.gate_up_swiglu(dense)"):
                    h, ws1 = moe_dense_gate_up(x, invert_permutation, expert_offset, self.wu.weight, self.wu.bias,
                                               return_workspace=True)
                return self._down_combine(h, ws1, expert_weights, invert_permutation, expert_offset)
        with _range("moe.route_select"):
            if router_logits is None and self.fused:
                routed = moe_route_select(x, self.gate.weight, E, k)     # decode-size batches: one launch
            if routed is not None:
                _, x_experts, expert_weights, invert_permutation, expert_offset = routed
            else:
                if router_logits is None:
                    router_logits = OPMX.router_gate(x, self.gate.weight)
                x_experts, expert_weights, invert_permutation, expert_offset = OPMX.moe_select(x, router_logits, E, k)
        if not self.fused:
            x13 = OPMX.swiglu(self.wu(x_experts, expert_offset))
            x_out = self.w2(x13, expert_offset)
            return OPMX.moe_reduce(x_out, expert_weights, invert_permutation, k)
        return self._experts(x_experts, expert_weights, invert_permutation, expert_offset)

    def _experts(self, x_experts, expert_weights, invert_permutation, expert_offset):
        """gate/up GEMM with SwiGLU epilogue -> down GEMM -> combine (+ exchange over TP)."""
        k = self.num_experts_per_token
        world = _world(self.proc_group)
        flat = x_experts.view(-1, self.hidden_dim)
        with _range("moe.gate_up_swiglu"):
            h, ws1 = moe_grouped_linear(flat, expert_offset, self.wu.weight, self.wu.bias, swiglu=True,
                                        zero_outside=False, return_workspace=True)
        return self._down_combine(h, ws1, expert_weights, invert_permutation, expert_offset)

    def _down_combine(self, h, ws1, expert_weights, invert_permutation, expert_offset):
        """down GEMM -> combine (+ exchange over TP) on the gate/up result h [T*k, I/tp]."""
        k = self.num_experts_per_token
        world = _world(self.proc_group)
        bias2 = self.w2.bias
        if bias2 is not None and world > 1 and dist.get_rank(group=self.proc_group) != 0:
            bias2 = None
        tokens = expert_weights.numel() // k
        if (world > 1 and self.overlap_chunks > 1 and self.hidden_dim % (8 * self.overlap_chunks) == 0
                and tokens * self.hidden_dim * h.element_size() >= OVERLAP_MIN_BYTES
                and not (self.peer_reduce_tokens >= tokens and self._peer_fits(tokens, h.dtype))):
            return self._down_combine_overlapped(h, expert_offset, expert_weights, invert_permutation, bias2, ws1)
        with _range("moe.down"):
            y, ws2 = moe_grouped_linear(h, expert_offset, self.w2.weight, bias2, zero_outside=False,
                                        return_workspace=True)
        self._last_workspaces = (ws1, ws2)
        self._mlp_ws = None
        return self._combine(y, expert_weights, invert_permutation)

    def _combine(self, y, expert_weights, invert_permutation):
        """combine (+ exchange over TP) of the down projection's rows y [T*k, H]."""
        k = self.num_experts_per_token
        world = _world(self.proc_group)
        with _range("moe.combine_allreduce"):
            if world > 1 and self.peer_reduce_tokens > 0:
                if self._peer is None:
                    from .peer_reduce import PeerCombine
                    self._peer = PeerCombine(self.proc_group, self.peer_reduce_tokens, self.hidden_dim, y.dtype,
                                             y.device, algorithm=self.peer_algorithm)
                if self._peer.fits(expert_weights.numel() // k, self.hidden_dim, y.dtype):
                    return self._peer.combine_allreduce(y, expert_weights, invert_permutation, k)
            out = OPMX.moe_reduce(y.view(*expert_weights.shape, -1), expert_weights, invert_permutation, k)
            if world > 1:
                if self._defer_allreduce:
                    self._pending.append(dist.all_reduce(out, group=self.proc_group, async_op=True))
                else:
                    dist.all_reduce(out, group=self.proc_group)
        return out

    def _forward_microbatched(self, x: torch.Tensor, router_logits, n_mb: int) -> torch.Tensor:
        """The block on n_mb runs of tokens, each followed by an asynchronous all-reduce of its
        result that overlaps the next run's kernels."""
        flat = x.reshape(-1, self.hidden_dim)
        logits = router_logits.reshape(flat.shape[0], -1) if router_logits is not None else None
        step = flat.shape[0] // n_mb
        self._defer_allreduce, self._pending = True, []
        try:
            outs = [self.forward(flat[i * step:(i + 1) * step],
                                 logits[i * step:(i + 1) * step] if logits is not None else None)
                    for i in range(n_mb)]
            for work in self._pending:
                work.wait()
        finally:
            self._defer_allreduce, self._pending = False, []
        return torch.cat(outs).view(*x.shape[:-1], self.hidden_dim)

    def _peer_fits(self, tokens: int, dtype) -> bool:
        from .peer_reduce import ONE_SHOT_LIMIT_BYTES
        return tokens * self.hidden_dim * torch.empty((), dtype=dtype).element_size() <= ONE_SHOT_LIMIT_BYTES

    def _down_combine_overlapped(self, h, expert_offset, expert_weights, invert_permutation, bias2, ws1):
        """Large batches under tensor parallelism: the down projection and the combine run per
        slice of the hidden columns, and the all-reduce of slice i (NCCL, on the process
        group's own stream) overlaps the GEMM of slice i+1.  Same sums as the unsliced path:
        every output element is produced by one GEMM tile, one combine and one all-reduce."""
        k = self.num_experts_per_token
        chunks = self.overlap_chunks
        Hc = self.hidden_dim // chunks
        plan = GemmPlan(stages=6)          # leaves shared memory on every SM for the collective's CTAs
        parts, works, spaces = [], [], [ws1]
        for c in range(chunks):
            w_c = self.w2.weight[:, c * Hc:(c + 1) * Hc, :]
            b_c = bias2[:, c * Hc:(c + 1) * Hc] if bias2 is not None else None
            with _range(f"moe.down[{c}]"):
                y_c, ws = moe_grouped_linear(h, expert_offset, w_c, b_c, zero_outside=False, plan=plan,
                                             return_workspace=True)
            with _range(f"moe.combine[{c}]"):
                o_c = OPMX.moe_reduce(y_c.view(*expert_weights.shape, Hc), expert_weights, invert_permutation, k)
            works.append(dist.all_reduce(o_c, group=self.proc_group, async_op=True))
            parts.append(o_c)
            spaces.append(ws)
        self._last_workspaces = tuple(spaces)
        for work in works:
            work.wait()
        return torch.cat(parts, dim=-1)

    def check(self) -> None:
        """Synchronises the device and raises (PmxError, status -6) if a kernel of the last
        step recorded a bounded wait that ran out: a pipeline barrier inside an expert GEMM,
        the grid barrier of the one-launch router + select, or a wait for a peer in the fused
        combine + all-reduce.  Without this call such a failure leaves undefined (GEMMs,
        select) or zero (all-reduce) rows behind silently; call it at step boundaries, or
        every N steps.  Not for use inside a CUDA graph capture."""
        from .torch_function.moe import grouped_linear_check, route_select_check
        for ws in self._last_workspaces:
            if ws is not None:
                grouped_linear_check(ws)
        if self._mlp_ws is not None:
            dense_mlp_check(self._mlp_ws, self.num_experts)
        route_select_check(device=self.gate.weight.device)
        if self._peer is not None:
            self._peer.check()


PATCHED_NAMES = ("moe_select", "moe_column_parallel_linear", "moe_row_parallel_linear", "moe_reduce",
                 "swiglu", "silu", "rms_norm", "skip_rms_norm",
                 "linear", "column_parallel_linear", "row_parallel_linear",
                 "dynamic_batching.multi_head_cache_attention")


def _resolve(module, dotted: str):
    *path, leaf = dotted.split(".")
    for part in path:
        module = getattr(module, part)
    return module, leaf


def patch_reference(opmx_module, names=PATCHED_NAMES) -> dict:
    """Rebind operators of an imported OPMX `torch_function` module to this implementation:
    the MoE entry points (the reference resolves them through that module at call time,
    Model.py:191-211 and ModelParallel.py:156,193), the normalisation in front of the block
    (ModelLayers.py:36-49), the dense linears around it (ModelLayers.py:69,
    ModelParallel.py:89,121) and the cache attention of decode steps (Model.py:103).  The
    attention replacement covers decode steps only: for any other call it hands over to the
    operator it replaced.  Returns {name: original function} so the caller can undo it
    (`for n, f in saved.items(): unpatch ...` or `unpatch_reference(opmx_module, saved)`)."""
    saved = {}
    for name in names:
        if name not in PATCHED_NAMES:
            raise ValueError(f"{name} is not an operator this package replaces")
        theirs_mod, leaf = _resolve(opmx_module, name)
        ours_mod, _ = _resolve(OPMX, name)
        original = getattr(theirs_mod, leaf)
        ours = getattr(ours_mod, leaf)
        saved[name] = original
        if name == "dynamic_batching.multi_head_cache_attention":
            def attention(*args, _ours=ours, _theirs=original, **kwargs):
                try:
                    return _ours(*args, **kwargs)
                except NotImplementedError:          # a prefill step, a paged or quantised cache, a mask
                    return _theirs(*args, **kwargs)
            setattr(theirs_mod, leaf, attention)
        else:
            setattr(theirs_mod, leaf, ours)
    return saved


def unpatch_reference(opmx_module, saved: dict) -> None:
    """Puts back what patch_reference() replaced."""
    for name, fn in saved.items():
        mod, leaf = _resolve(opmx_module, name)
        setattr(mod, leaf, fn)
