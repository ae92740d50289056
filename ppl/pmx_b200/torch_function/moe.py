"""The OPMX mixture-of-experts operators on B200.

Same call signatures, output layouts, dtypes and ONNX custom-op export as the
reference operators; `forward` allocates the outputs and hands raw pointers to
the CUDA library through its C ABI.  Tensors must live on a CUDA device: there
is no CPU implementation behind these functions (during ONNX export the
forwards only return correctly shaped placeholders, as the reference does).

Reference: torch_function/MoeSelect.py, MoeColumnParallelLinear.py,
MoeRowParallelLinear.py, MoeReduce.py, SwiGLU.py, SiLU.py.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .. import _cabi
from .._cabi import lib, check, ptr, stream_of, workspace, DTYPE_CODE


def _require_cuda(name: str, **tensors) -> None:
    for key, t in tensors.items():
        if t is not None and not t.is_cuda:
            raise RuntimeError(f"{name}: `{key}` is on {t.device}; this implementation runs on CUDA "
                               "devices only and has no CPU fallback")


def _dtype_code(name: str, t: torch.Tensor) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise TypeError(f"{name}: dtype {t.dtype} is not supported (float16, bfloat16, float32)") from None


def _group_size(proc_group) -> int:
    if proc_group is None or not dist.is_available() or not dist.is_initialized():
        return 1
    return dist.get_world_size(group=proc_group)


def _offsets_on(expert_offset: torch.Tensor, device, num_experts: int) -> torch.Tensor:
    if expert_offset.numel() != num_experts + 1:
        raise ValueError(f"expert_offset has {expert_offset.numel()} entries, expected num_experts+1 = {num_experts + 1}")
    return expert_offset.to(device=device, dtype=torch.int64).contiguous()


# --------------------------------------------------------------------------- select
class MoeSelect(torch.autograd.Function):
    """opmx::MoeSelect (torch_function/MoeSelect.py:5-64)."""

    @staticmethod
    def symbolic(g, X, scores, num_experts: int, num_experts_per_token: int):
        return g.op("opmx::MoeSelect", X, scores, num_experts_i=num_experts,
                    num_experts_per_token_i=num_experts_per_token, outputs=4)

    @staticmethod
    def forward(ctx, X: torch.Tensor, scores: torch.Tensor, num_experts: int, num_experts_per_token: int):
        k = int(num_experts_per_token)
        lead = tuple(X.shape[:-1])
        H = X.shape[-1]
        if torch.onnx.is_in_onnx_export():
            # placeholders in the order of the real outputs (the reference
            # returns them permuted at MoeSelect.py:35, which only shuffles the
            # traced type metadata)
            return (torch.zeros(*lead, k, H, dtype=X.dtype, device=X.device),
                    torch.zeros(*lead, k, dtype=scores.dtype, device=X.device),
                    torch.zeros(*lead, k, dtype=torch.int64, device=X.device),
                    torch.zeros(num_experts + 1, dtype=torch.int64, device=X.device))
        _require_cuda("moe_select", X=X, scores=scores)
        if scores.shape[-1] != num_experts or tuple(scores.shape[:-1]) != lead:
            raise ValueError(f"moe_select: scores shape {tuple(scores.shape)} does not match X {tuple(X.shape)} "
                             f"with {num_experts} experts")
        if scores.dtype != X.dtype:
            raise TypeError("moe_select: X and scores must have the same dtype")
        if not 0 < k <= num_experts:
            raise ValueError(f"moe_select: num_experts_per_token={k} out of range for {num_experts} experts")
        T = 1
        for d in lead:
            T *= d
        if T == 0 or H == 0:
            raise ValueError("moe_select: needs at least one token")
        code = _dtype_code("moe_select", X)
        x2 = X.contiguous().view(T, H)
        s2 = scores.contiguous().view(T, num_experts)
        dev = X.device
        xp = torch.empty(*lead, k, H, dtype=X.dtype, device=dev)
        w = torch.empty(*lead, k, dtype=scores.dtype, device=dev)
        inv = torch.empty(*lead, k, dtype=torch.int64, device=dev)
        off = torch.empty(num_experts + 1, dtype=torch.int64, device=dev)
        nbytes = lib.pmx_moe_select_workspace_bytes(T, num_experts, k)
        ws = workspace(nbytes, dev)
        with torch.cuda.device(dev):
            check(lib.pmx_moe_select(ptr(x2), ptr(s2), ptr(xp), ptr(w), ptr(inv), ptr(off), T, H,
                                     num_experts, k, code, ptr(ws), ws.numel(), stream_of(X)))
        return xp, w, inv, off


def moe_select(X: torch.Tensor, scores: torch.Tensor, num_experts: int, num_experts_per_token: int):
    """-> (X_expand_permute [*,k,H], expert_weights [*,k], invert_permutation [*,k] int64,
    expert_offset [E+1] int64); signature of torch_function/MoeSelect.py:67-70."""
    return MoeSelect.apply(X, scores, num_experts, num_experts_per_token)


def _route_select_workspace(nbytes: int, dev, given):
    if given is None:
        return _cabi.barrier_workspace(nbytes, dev)
    if given.device != dev or given.numel() * given.element_size() < nbytes:
        raise ValueError(f"workspace must hold {nbytes} bytes on {dev} (first 64 bytes zero before its first use)")
    return given


def route_select_check(workspace: torch.Tensor | None = None, device=None) -> None:
    """Synchronises and raises if the grid barrier of an earlier moe_route_select /
    moe_norm_route_select call on this workspace (default: the device's own) gave up;
    the barrier words are cleared so that the next call starts clean."""
    if workspace is not None:
        ws = workspace
    else:
        index = torch.device(device).index if device is not None else None
        ws = _cabi._barrier_ws.get((torch.cuda.current_device() if index is None else index, "route"))
    if ws is None:
        return
    with torch.cuda.device(ws.device):
        status = lib.pmx_moe_route_select_check(ptr(ws), stream_of(ws))
        if status != 0:
            text = lib.pmx_moe_last_error().decode()
            ws[:64].zero_()
            raise _cabi.PmxError(status, text)


def moe_route_select(X: torch.Tensor, W_router: torch.Tensor, num_experts: int, num_experts_per_token: int,
                     workspace: torch.Tensor | None = None, gather: bool = True):
    """Router gate and moe_select in one launch for decode-size batches:
    scores = X @ W_router.T (Linear.py:24-33 as called at Model.py:188), then
    MoeSelect (MoeSelect.py:36-64) on those scores.
    -> (scores [*,E], X_expand_permute, expert_weights, invert_permutation, expert_offset),
    or None when the shape is outside what the fused kernel covers (more than 1024
    tokens, more than 64 experts, ...): call a linear and moe_select then.
    `workspace`: see _cabi.barrier_workspace (default: one kept buffer per device).
    gather=False: X_expand_permute is not produced (None is returned in its place), for the
    dense gate/up projection that reads the un-permuted tokens."""
    _require_cuda("moe_route_select", X=X, W_router=W_router)
    k, E = int(num_experts_per_token), int(num_experts)
    lead, H = tuple(X.shape[:-1]), X.shape[-1]
    if tuple(W_router.shape) != (E, H) or W_router.dtype != X.dtype:
        raise ValueError(f"W_router must be [{E}, {H}] in X's dtype")
    T = 1
    for d in lead:
        T *= d
    code = _dtype_code("moe_route_select", X)
    nbytes = lib.pmx_moe_route_select_workspace_bytes(T, H, E, k, code) if T > 0 else 0
    if nbytes == 0:
        return None
    dev = X.device
    x2 = X.contiguous().view(T, H)
    wr = W_router.contiguous()
    scores = torch.empty(*lead, E, dtype=X.dtype, device=dev)
    xp = torch.empty(*lead, k, H, dtype=X.dtype, device=dev) if gather else None
    w = torch.empty(*lead, k, dtype=X.dtype, device=dev)
    inv = torch.empty(*lead, k, dtype=torch.int64, device=dev)
    off = torch.empty(E + 1, dtype=torch.int64, device=dev)
    ws = _route_select_workspace(nbytes, dev, workspace)
    with torch.cuda.device(dev):
        check(lib.pmx_moe_route_select(ptr(x2), ptr(wr), ptr(scores), ptr(xp), ptr(w), ptr(inv), ptr(off), T, H,
                                       E, k, code, ptr(ws), ws.numel(), stream_of(X)))
    return scores, xp, w, inv, off


def moe_norm_route_select(X: torch.Tensor, SkipIn: torch.Tensor | None, norm_weight: torch.Tensor, eps: float,
                          W_router: torch.Tensor, num_experts: int, num_experts_per_token: int,
                          workspace: torch.Tensor | None = None):
    """skip_rms_norm -> router gate -> moe_select in one launch for decode-size batches
    (RMSNorm.py:42-56, Linear.py:24-33 and MoeSelect.py:36-64 as called at Model.py:261,188,191).
    -> (SkipOut, scores, X_expand_permute, expert_weights, invert_permutation, expert_offset),
    X_expand_permute holding rows of the normalised input; SkipOut is X itself when SkipIn is
    None.  Returns None when the shape is outside what the fused kernel covers."""
    _require_cuda("moe_norm_route_select", X=X, SkipIn=SkipIn, norm_weight=norm_weight, W_router=W_router)
    k, E = int(num_experts_per_token), int(num_experts)
    lead, H = tuple(X.shape[:-1]), X.shape[-1]
    if tuple(W_router.shape) != (E, H) or W_router.dtype != X.dtype:
        raise ValueError(f"W_router must be [{E}, {H}] in X's dtype")
    if tuple(norm_weight.shape) != (H,) or norm_weight.dtype != X.dtype:
        raise ValueError(f"norm_weight must be [{H}] in X's dtype")
    if SkipIn is not None and (SkipIn.shape != X.shape or SkipIn.dtype != X.dtype):
        raise ValueError("SkipIn must match X in shape and dtype")
    T = 1
    for d in lead:
        T *= d
    code = _dtype_code("moe_norm_route_select", X)
    nbytes = lib.pmx_moe_norm_route_select_workspace_bytes(T, H, E, k, code) if T > 0 else 0
    if nbytes == 0:
        return None
    dev = X.device
    x2 = X.contiguous().view(T, H)
    s2 = SkipIn.contiguous().view(T, H) if SkipIn is not None else None
    skip_out = torch.empty_like(x2) if SkipIn is not None else None
    scores = torch.empty(*lead, E, dtype=X.dtype, device=dev)
    xp = torch.empty(*lead, k, H, dtype=X.dtype, device=dev)
    w = torch.empty(*lead, k, dtype=X.dtype, device=dev)
    inv = torch.empty(*lead, k, dtype=torch.int64, device=dev)
    off = torch.empty(E + 1, dtype=torch.int64, device=dev)
    ws = _route_select_workspace(nbytes, dev, workspace)
    with torch.cuda.device(dev):
        check(lib.pmx_moe_norm_route_select(ptr(x2), ptr(s2), ptr(norm_weight.contiguous()), float(eps),
                                            ptr(W_router.contiguous()), ptr(skip_out), ptr(scores), ptr(xp), ptr(w),
                                            ptr(inv), ptr(off), T, H, E, k, code, ptr(ws), ws.numel(), stream_of(X)))
    return (X if skip_out is None else skip_out.view_as(X)), scores, xp, w, inv, off


# --------------------------------------------------------------------------- grouped linear
def moe_grouped_linear(X: torch.Tensor, expert_offset: torch.Tensor, W: torch.Tensor,
                       B: torch.Tensor | None = None, *, swiglu: bool = False, beta: float = 1.0,
                       zero_outside: bool = True, plan: _cabi.GemmPlan | None = None,
                       return_workspace: bool = False):
    """Y[r] = X[r] @ W[e].T (+ B[e]) for rows r in [expert_offset[e], expert_offset[e+1]).

    X [*,K], W [E,N,K], B [E,N] or None -> Y [*,N]; with swiglu=True W holds the
    gate rows then the up rows and Y is [*,N/2] = up * gate * sigmoid(beta*gate).
    expert_offset=None (E == 1 only): the one expert owns all rows, a dense linear.
    The shared core of moe_column_parallel_linear and moe_row_parallel_linear
    (the loops at MoeColumnParallelLinear.py:61-67 and MoeRowParallelLinear.py:47-53).
    """
    _require_cuda("moe_grouped_linear", X=X, W=W, B=B)
    if W.dim() != 3:
        raise ValueError("W must be [num_experts, out_features, in_features]")
    E, N, K = W.shape
    if X.shape[-1] != K:
        raise ValueError(f"X has {X.shape[-1]} input features, W expects {K}")
    if W.dtype != X.dtype or (B is not None and B.dtype != X.dtype):
        raise TypeError("X, W and B must have the same dtype")
    if B is not None and tuple(B.shape) != (E, N):
        raise ValueError(f"B must be [{E}, {N}]")
    code = _dtype_code("moe_grouped_linear", X)
    dev = X.device
    lead = tuple(X.shape[:-1])
    M = 1
    for d in lead:
        M *= d
    n_out = N // 2 if swiglu else N
    y = torch.empty(*lead, n_out, dtype=X.dtype, device=dev)
    if M == 0:
        return (y, None) if return_workspace else y
    x2 = X.contiguous().view(M, K)
    # W may be a window of the feature rows of a wider weight tensor (W_full[:, n0:n1, :]):
    # it is used in place, with the distance between experts passed as a row pitch
    pitch = 0
    if (not W.is_contiguous() and not swiglu and W.stride(2) == 1 and W.stride(1) == K and E > 1
            and W.stride(0) % K == 0 and W.stride(0) // K >= N and (B is None or B.is_contiguous() is False)):
        pitch = W.stride(0) // K
        w = W
        b = B
        if b is not None and not (b.stride(1) == 1 and b.stride(0) == pitch):
            raise ValueError("a bias passed with a window of W must be the same window of the full bias")
    else:
        w = W.contiguous()
        b = B.contiguous() if B is not None else None
    if pitch:
        if plan is None:
            plan = _cabi.GemmPlan()
        else:
            plan = _cabi.GemmPlan.from_buffer_copy(plan)
        plan.w_expert_pitch = pitch
    if expert_offset is None and E != 1:
        raise ValueError("expert_offset may be None only for a single expert")
    off = _offsets_on(expert_offset, dev, E) if expert_offset is not None else None
    epi = _cabi.EPILOGUE_SWIGLU if swiglu else _cabi.EPILOGUE_NONE
    plan_ref = C.byref(plan) if plan is not None else None
    nbytes = lib.pmx_moe_grouped_linear_workspace_bytes(M, N, K, E, code, epi, plan_ref)
    if nbytes == 0:
        raise _cabi.PmxError(-1, lib.pmx_moe_last_error().decode() or "grouped_linear: invalid arguments")
    ws = workspace(nbytes, dev)
    with torch.cuda.device(dev):
        check(lib.pmx_moe_grouped_linear(ptr(x2), ptr(off), ptr(w), ptr(b), ptr(y), M, N, K, E, code, epi,
                                         float(beta), 1 if zero_outside else 0, plan_ref, ptr(ws),
                                         ws.numel(), stream_of(X)))
    return (y, ws) if return_workspace else y


def dense_gate_up_covers(T: int, W: torch.Tensor, k: int) -> bool:
    """Whether moe_dense_gate_up takes this shape AND pays.  Measured on B200 (Mixtral shapes,
    64 tokens): hiding the router saves 6-7 us per step, but the larger token tile (all T tokens
    instead of an expert's share) costs one ring stage, about 5 % of the weight-streaming time,
    and every expert's weights are read even if no token chose it.  So: at most 64 tokens, a
    launch of at most two 128-row weight tiles per working CTA (the thin shards of tensor
    parallelism, where the router is a tenth of the step), and a chance of an unused expert,
    ((E-k)/E)^T, below 2 %."""
    E, N, K = W.shape
    code = DTYPE_CODE.get(W.dtype)
    if T > 64 or code is None or not lib.pmx_moe_dense_gate_up_covers(T, N, K, E, k, code):
        return False
    if E * ((N // 2 + 127) // 128) > 2 * 128:
        return False
    return ((E - k) / E) ** T < 0.02


def moe_dense_gate_up(X: torch.Tensor, invert_permutation: torch.Tensor, expert_offset: torch.Tensor,
                      W: torch.Tensor, B: torch.Tensor | None = None, beta: float = 1.0,
                      return_workspace: bool = False):
    """H[r] = SwiGLU(X[t] @ W[e].T (+ B[e])) for every (token t, chosen expert e), r = the row of
    that pair in the expert-sorted order: what moe_column_parallel_linear + swiglu give for
    the rows moe_select gathers (MoeColumnParallelLinear.py:58-69, SwiGLU.py:15-16), computed
    from the un-permuted X [T,K].  Launch it directly behind moe_route_select on the same
    stream: the weight streaming then overlaps the router (see pmx_moe_dense_gate_up)."""
    _require_cuda("moe_dense_gate_up", X=X, W=W, B=B, invert_permutation=invert_permutation)
    E, N, K = W.shape
    T = X.numel() // K
    k = invert_permutation.shape[-1]
    code = _dtype_code("moe_dense_gate_up", X)
    if W.dtype != X.dtype or (B is not None and B.dtype != X.dtype):
        raise TypeError("X, W and B must have the same dtype")
    dev = X.device
    h = torch.empty(T * k, N // 2, dtype=X.dtype, device=dev)
    ws = workspace(256, dev)
    x2, w = X.contiguous().view(T, K), W.contiguous()
    b = B.contiguous() if B is not None else None
    inv = invert_permutation.contiguous()
    off = _offsets_on(expert_offset, dev, E)
    with torch.cuda.device(dev):
        check(lib.pmx_moe_dense_gate_up(ptr(x2), ptr(inv), ptr(off), ptr(w), ptr(b), ptr(h), T, N, K, E, k, code,
                                        float(beta), ptr(ws), ws.numel(), stream_of(X)))
    return (h, ws) if return_workspace else h


ONE_LAUNCH_MAX_TILES = 2 * 128     # 128-row gate/up tiles of all experts up to which moe_dense_mlp is used
ONE_LAUNCH_MAX_TOKENS = 128        # ... and tokens (the kernel's own limit)
ONE_LAUNCH_MAX_UNUSED = 0.15       # ... and chance that an expert has no token (its weights are read anyway)


def dense_mlp_covers(T: int, Wu: torch.Tensor, W2: torch.Tensor, k: int) -> bool:
    """Whether moe_dense_mlp takes this shape and pays: decode batches of at most 128 tokens,
    without bias, up to ONE_LAUNCH_MAX_TILES gate/up tiles (the tp-4 and tp-8 shards of Mixtral),
    a chance of an unused expert, ((E-k)/E)^T, below 15 % (every expert's weights are read).
    Measured on B200, 1/8 shard of the Mixtral layer, step with one launch against two:
    8 tokens 71.7 / 88.9 us, 64 tokens 79.1 / 92.5 us, 128 tokens 88.5 / 102.5 us; 1/4 shard
    125.4 / 133.9, 132.8 / 142.5 and 150.2 / 154.0 us; at full size two launches win."""
    E, N, H = Wu.shape
    code = DTYPE_CODE.get(Wu.dtype)
    if code is None or tuple(W2.shape) != (E, H, N // 2) or W2.dtype != Wu.dtype:
        return False
    if (T > ONE_LAUNCH_MAX_TOKENS or E * ((N // 2 + 127) // 128) > ONE_LAUNCH_MAX_TILES
            or ((E - k) / E) ** T >= ONE_LAUNCH_MAX_UNUSED):
        return False
    return bool(lib.pmx_moe_dense_mlp_covers(T, N, H, E, k, code))


def moe_dense_mlp(X: torch.Tensor, invert_permutation: torch.Tensor, expert_offset: torch.Tensor,
                  Wu: torch.Tensor, W2: torch.Tensor, beta: float = 1.0, workspace: torch.Tensor | None = None,
                  return_workspace: bool = False):
    """Y[r] = SwiGLU(X[t] @ Wu[e].T) @ W2[e].T for every (token t, chosen expert e), r = the row of
    that pair in the expert-sorted order: moe_column_parallel_linear + swiglu +
    moe_row_parallel_linear (before its all-reduce) of the reference for the rows moe_select
    gathers (Model.py:198-205), from the un-permuted X [T,H], in one launch (see
    pmx_moe_dense_mlp).  -> Y [T*k, H].  Launch it directly behind moe_route_select on the
    same stream.  `workspace`: see _cabi.barrier_workspace (default: one kept buffer per device)."""
    _require_cuda("moe_dense_mlp", X=X, Wu=Wu, W2=W2, invert_permutation=invert_permutation)
    E, N, H = Wu.shape
    T = X.numel() // H
    k = invert_permutation.shape[-1]
    code = _dtype_code("moe_dense_mlp", X)
    if Wu.dtype != X.dtype or W2.dtype != X.dtype:
        raise TypeError("X, Wu and W2 must have the same dtype")
    if tuple(W2.shape) != (E, H, N // 2):
        raise ValueError(f"W2 must be [{E}, {H}, {N // 2}], got {tuple(W2.shape)}")
    dev = X.device
    h = torch.empty(T * k, N // 2, dtype=X.dtype, device=dev)
    y = torch.empty(T * k, H, dtype=X.dtype, device=dev)
    nbytes = lib.pmx_moe_dense_mlp_workspace_bytes(E)
    ws = workspace if workspace is not None else _cabi.barrier_workspace(nbytes, dev, kind="mlp")
    x2, wu, w2 = X.contiguous().view(T, H), Wu.contiguous(), W2.contiguous()
    inv = invert_permutation.contiguous()
    off = _offsets_on(expert_offset, dev, E)
    with torch.cuda.device(dev):
        check(lib.pmx_moe_dense_mlp(ptr(x2), ptr(inv), ptr(off), ptr(wu), ptr(w2), ptr(h), ptr(y), T, N, H, E, k,
                                    code, float(beta), ptr(ws), ws.numel(), stream_of(X)))
    return (y, ws) if return_workspace else y


def dense_mlp_check(ws: torch.Tensor, num_experts: int) -> None:
    """Synchronises and raises if the moe_dense_mlp launch that used `ws` recorded a wait that ran out."""
    out = (C.c_int32 * 4)()
    with torch.cuda.device(ws.device):
        check(lib.pmx_moe_dense_mlp_check(ptr(ws), int(num_experts), C.byref(out), stream_of(ws)))


def grouped_linear_check(ws: torch.Tensor) -> None:
    """Synchronises and raises if the launch that used `ws` recorded a failed self-check."""
    out = (C.c_int32 * 4)()
    with torch.cuda.device(ws.device):
        check(lib.pmx_moe_grouped_linear_check(ptr(ws), C.byref(out), stream_of(ws)))


class MoeColumnParallelLinear(torch.autograd.Function):
    """opmx::MoeColumnParallelLinear (torch_function/MoeColumnParallelLinear.py:7-81)."""

    @staticmethod
    def symbolic(g, X, expert_offset, W, B, proc_group, num_experts: int, in_features: int,
                 out_features: int, gather_output: bool = True):
        attrs = dict(num_experts_i=num_experts, in_features_i=in_features, out_features_i=out_features,
                     gather_output_i=gather_output)
        if B is not None:
            return g.op("opmx::MoeColumnParallelLinear", X, expert_offset, W, B, bias_term_i=True, **attrs)
        return g.op("opmx::MoeColumnParallelLinear", X, expert_offset, W, bias_term_i=False, **attrs)

    @staticmethod
    def forward(ctx, X, expert_offset, W, B, proc_group, num_experts: int, in_features: int,
                out_features: int, gather_output: bool = True):
        assert X.shape[-1] == in_features, "X.shape is {}, in_features is {}".format(X.shape, in_features)
        world = _group_size(proc_group)
        if torch.onnx.is_in_onnx_export():
            part = torch.zeros(*X.shape[:-1], W.shape[1], dtype=W.dtype, device=X.device)
            if gather_output and world > 1:
                return torch.cat([part] * world, dim=-1)
            return part
        if W.shape[0] != num_experts:
            raise ValueError(f"W has {W.shape[0]} experts, num_experts={num_experts}")
        y = moe_grouped_linear(X, expert_offset, W, B)
        if gather_output and world > 1:
            parts = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(parts, y, group=proc_group)
            y = torch.cat(parts, dim=-1).contiguous()
        return y


def moe_column_parallel_linear(X, expert_offset, W, B, proc_group, num_experts: int, in_features: int,
                               out_features: int, gather_output: bool = True) -> torch.Tensor:
    """Signature of torch_function/MoeColumnParallelLinear.py:84-93.  W is this rank's
    [E, out_features/tp, in_features] shard; the output keeps X's dtype and device."""
    return MoeColumnParallelLinear.apply(X, expert_offset, W, B, proc_group, num_experts, in_features,
                                         out_features, gather_output)


class MoeRowParallelLinear(torch.autograd.Function):
    """opmx::MoeRowParallelLinear (torch_function/MoeRowParallelLinear.py:8-62)."""

    @staticmethod
    def symbolic(g, X, expert_offset, W, B, proc_group, num_experts: int, in_features: int,
                 out_features: int, input_is_parallel: bool = False):
        attrs = dict(num_experts_i=num_experts, in_features_i=in_features, out_features_i=out_features,
                     input_is_parallel_i=input_is_parallel)
        if B is not None:
            return g.op("opmx::MoeRowParallelLinear", X, expert_offset, W, B, bias_term_i=True, **attrs)
        return g.op("opmx::MoeRowParallelLinear", X, expert_offset, W, bias_term_i=False, **attrs)

    @staticmethod
    def forward(ctx, X, expert_offset, W, B, proc_group, num_experts: int, in_features: int,
                out_features: int, input_is_parallel: bool = False):
        if torch.onnx.is_in_onnx_export():
            return torch.zeros(*X.shape[:-1], W.shape[1], dtype=W.dtype, device=X.device)
        if W.shape[0] != num_experts:
            raise ValueError(f"W has {W.shape[0]} experts, num_experts={num_experts}")
        world = _group_size(proc_group)
        # X is taken as already split along K (the reference ignores
        # input_is_parallel too, MoeRowParallelLinear.py:44-53).  The bias is
        # per expert and must enter the sum once: only group rank 0 adds it.
        # (The reference's `output + B` at :59-60 broadcasts [E,N] against the
        # row dimension and is not per expert; the operator spec asks for B:(E,N).)
        bias = B
        if B is not None and world > 1 and dist.get_rank(group=proc_group) != 0:
            bias = None
        y = moe_grouped_linear(X, expert_offset, W, bias)
        if world > 1:
            dist.all_reduce(y, group=proc_group)
        return y


def moe_row_parallel_linear(X, expert_offset, W, B, proc_group, num_experts: int, in_features: int,
                            out_features: int, input_is_parallel: bool = False) -> torch.Tensor:
    """Signature of torch_function/MoeRowParallelLinear.py:65-74.  W is this rank's
    [E, out_features, in_features/tp] shard; partial sums are all-reduced over proc_group."""
    return MoeRowParallelLinear.apply(X, expert_offset, W, B, proc_group, num_experts, in_features,
                                      out_features, input_is_parallel)


# --------------------------------------------------------------------------- reduce
class MoeReduce(torch.autograd.Function):
    """opmx::MoeReduce (torch_function/MoeReduce.py:4-26)."""

    @staticmethod
    def symbolic(g, Y, expert_weights, invert_permutation, num_experts_per_token: int):
        out = g.op("opmx::MoeReduce", Y, expert_weights, invert_permutation,
                   num_experts_per_token_i=num_experts_per_token)
        return out.setTypeAs(Y)

    @staticmethod
    def forward(ctx, Y, expert_weights, invert_permutation, num_experts_per_token: int):
        k = int(num_experts_per_token)
        N = Y.shape[-1]
        lead = tuple(expert_weights.shape[:-1])
        if torch.onnx.is_in_onnx_export():
            return torch.zeros(*lead, N, dtype=Y.dtype, device=Y.device)
        _require_cuda("moe_reduce", Y=Y, expert_weights=expert_weights, invert_permutation=invert_permutation)
        if expert_weights.shape[-1] != k or tuple(invert_permutation.shape) != tuple(expert_weights.shape):
            raise ValueError("moe_reduce: expert_weights and invert_permutation must be [*, num_experts_per_token]")
        T = expert_weights.numel() // k
        if Y.numel() != T * k * N:
            raise ValueError(f"moe_reduce: Y has {Y.numel()} elements, expected {T}*{k}*{N}")
        code = _dtype_code("moe_reduce", Y)
        out = torch.empty(*lead, N, dtype=Y.dtype, device=Y.device)
        if T == 0:
            return out
        y2 = Y.contiguous()
        w = expert_weights.to(Y.dtype).contiguous()
        inv = invert_permutation.to(torch.int64).contiguous()
        with torch.cuda.device(Y.device):
            check(lib.pmx_moe_reduce(ptr(y2), ptr(w), ptr(inv), ptr(out), T, k, N, code, stream_of(Y)))
        return out


def moe_reduce(Y, expert_weights, invert_permutation, num_experts_per_token: int):
    """Signature of torch_function/MoeReduce.py:29-32.  -> [*, N] in Y's dtype."""
    return MoeReduce.apply(Y, expert_weights, invert_permutation, num_experts_per_token)


# --------------------------------------------------------------------------- activations
class SwiGLU(torch.autograd.Function):
    """opmx::SwiGLU (torch_function/SwiGLU.py:4-17)."""

    @staticmethod
    def symbolic(g, X, beta: float = 1.0):
        return g.op("opmx::SwiGLU", X, beta_f=beta)

    @staticmethod
    def forward(ctx, X, beta: float = 1.0):
        D = X.shape[-1]
        if torch.onnx.is_in_onnx_export():
            return torch.zeros(*X.shape[:-1], D // 2, dtype=X.dtype, device=X.device)
        _require_cuda("swiglu", X=X)
        if D % 2:
            raise ValueError("swiglu: the last dimension must be even")
        code = _dtype_code("swiglu", X)
        y = torch.empty(*X.shape[:-1], D // 2, dtype=X.dtype, device=X.device)
        M = X.numel() // D if D else 0
        if M == 0:
            return y
        x2 = X.contiguous()
        with torch.cuda.device(X.device):
            check(lib.pmx_swiglu(ptr(x2), ptr(y), M, D, float(beta), code, stream_of(X)))
        return y


def swiglu(X: torch.Tensor, beta: float = 1.0):
    """Signature of torch_function/SwiGLU.py:20-21."""
    return SwiGLU.apply(X, beta)


class SiLU(torch.autograd.Function):
    """opmx::SiLU (torch_function/SiLU.py:4-21)."""

    @staticmethod
    def symbolic(g, X, gate=None):
        y = g.op("opmx::SiLU", X, gate) if gate is not None else g.op("opmx::SiLU", X)
        return y.setTypeAs(X)

    @staticmethod
    def forward(ctx, X, gate=None):
        if torch.onnx.is_in_onnx_export():
            return X
        _require_cuda("silu", X=X, gate=gate)
        if gate is not None and (gate.shape != X.shape or gate.dtype != X.dtype):
            raise ValueError("silu: gate must match X in shape and dtype")
        code = _dtype_code("silu", X)
        y = torch.empty_like(X, memory_format=torch.contiguous_format)
        if X.numel() == 0:
            return y
        x2 = X.contiguous()
        g2 = gate.contiguous() if gate is not None else None
        with torch.cuda.device(X.device):
            check(lib.pmx_silu(ptr(x2), ptr(g2), ptr(y), X.numel(), code, stream_of(X)))
        return y


def silu(X: torch.Tensor, gate: torch.Tensor = None):
    """Signature of torch_function/SiLU.py:24-25."""
    return SiLU.apply(X, gate)


# --------------------------------------------------------------------------- normalisation in front of the block
def _rms_norm_launch(name, X, weight, SkipIn, axis, eps):
    _require_cuda(name, X=X, weight=weight, SkipIn=SkipIn)
    H = X.shape[-1]
    if axis not in (-1, X.dim() - 1):
        raise ValueError(f"{name}: only the last axis is supported (axis={axis})")
    if tuple(weight.shape) != (H,) or weight.dtype != X.dtype:
        raise ValueError(f"{name}: weight must be [{H}] in X's dtype")
    if SkipIn is not None and (SkipIn.shape != X.shape or SkipIn.dtype != X.dtype):
        raise ValueError(f"{name}: SkipIn must match X in shape and dtype")
    code = _dtype_code(name, X)
    M = X.numel() // H if H else 0
    y = torch.empty_like(X, memory_format=torch.contiguous_format)
    skip_out = torch.empty_like(y) if SkipIn is not None else None
    if M > 0:
        x2, w2 = X.contiguous(), weight.contiguous()
        s2 = SkipIn.contiguous() if SkipIn is not None else None
        with torch.cuda.device(X.device):
            check(lib.pmx_skip_rms_norm(ptr(x2), ptr(s2), ptr(w2), ptr(y), ptr(skip_out), M, H, float(eps), code,
                                        stream_of(X)))
    return y, skip_out


class RMSNorm(torch.autograd.Function):
    """opmx::RMSNorm without skip (torch_function/RMSNorm.py:4-24)."""

    @staticmethod
    def symbolic(g, X, weight, axis: int = -1, eps: float = 1e-5):
        return g.op("opmx::RMSNorm", X, weight, axis_i=axis, eps_f=eps, skip_term_i=False).setTypeAs(X)

    @staticmethod
    def forward(ctx, X, weight, axis: int = -1, eps: float = 1e-5):
        if torch.onnx.is_in_onnx_export():
            return X
        return _rms_norm_launch("rms_norm", X, weight, None, axis, eps)[0]


class SkipRMSNorm(torch.autograd.Function):
    """opmx::RMSNorm with skip_term (torch_function/RMSNorm.py:27-56)."""

    @staticmethod
    def symbolic(g, X, weight, SkipIn=None, axis: int = -1, eps: float = 1e-5):
        args = (X, weight) if SkipIn is None else (X, weight, SkipIn)
        Y, SkipOut = g.op("opmx::RMSNorm", *args, axis_i=axis, eps_f=eps, skip_term_i=True, outputs=2)
        return Y.setTypeAs(X), SkipOut.setTypeAs(X)

    @staticmethod
    def forward(ctx, X, weight, SkipIn=None, axis: int = -1, eps: float = 1e-5):
        if torch.onnx.is_in_onnx_export():
            return X, X
        y, skip_out = _rms_norm_launch("skip_rms_norm", X, weight, SkipIn, axis, eps)
        return y, (X if skip_out is None else skip_out)


def rms_norm(X: torch.Tensor, weight: torch.Tensor, axis: int = -1, eps: float = 1e-5) -> torch.Tensor:
    """Signature of torch_function/RMSNorm.py:59-61."""
    return RMSNorm.apply(X, weight, axis, eps)


def skip_rms_norm(X: torch.Tensor, weight: torch.Tensor, SkipIn: torch.Tensor = None, axis: int = -1,
                  eps: float = 1e-5):
    """Signature of torch_function/RMSNorm.py:64-66.  -> (Y, SkipOut); SkipOut is X + SkipIn
    (X itself when SkipIn is None), the residual stream the next layer receives."""
    return SkipRMSNorm.apply(X, weight, SkipIn, axis, eps)
