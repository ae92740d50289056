"""ctypes binding of libpmx_moe_b200.so (declared in include/pmx_moe.h).

The library is the only compute backend of this package: if it cannot be
loaded, importing any operator fails with an ImportError that says how to build
it.  There is no CPU path behind these calls.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libpmx_moe_b200.so")

DTYPE_CODE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
ABI_VERSION = 3
EPILOGUE_NONE, EPILOGUE_SWIGLU = 0, 1
GEMM_AUTO, GEMM_TC_TOKENS_M, GEMM_TC_WEIGHTS_M, GEMM_SIMT, GEMM_TC_TOKENS_M_PAIRED = 0, 1, 2, 3, 4


class GemmPlan(C.Structure):
    """Mirror of pmx_gemm_plan."""
    _fields_ = [("kernel", C.c_int32), ("tile_feat", C.c_int32), ("tile_tok", C.c_int32),
                ("split_k", C.c_int32), ("stages", C.c_int32), ("max_ctas", C.c_int32), ("stream_k", C.c_int32),
                ("cta_cap", C.c_int32), ("full_rounds", C.c_int32), ("balance", C.c_int32), ("w_expert_pitch", C.c_int32),
                ("l2_prefetch", C.c_int32)]


class PmxError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"pmx_moe status {status}: {text}")
        self.status = status


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m ppl.pmx_b200.build` "
            "(needs nvcc with sm_100a support).  This package has no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64, sz, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t, C.c_float
    plan_p = C.POINTER(GemmPlan)
    sig = {
        "pmx_moe_abi_version": (C.c_int, []),
        "pmx_moe_last_error": (C.c_char_p, []),
        "pmx_moe_status_string": (C.c_char_p, [C.c_int]),
        "pmx_moe_kernel_launches": (C.c_longlong, []),
        "pmx_moe_select_workspace_bytes": (sz, [i64, i32, i32]),
        "pmx_moe_select": (C.c_int, [vp, vp, vp, vp, vp, vp, i64, i64, i32, i32, i32, vp, sz, vp]),
        "pmx_moe_route_select_workspace_bytes": (sz, [i64, i64, i32, i32, i32]),
        "pmx_moe_route_select": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, i32, i32, vp, sz, vp]),
        "pmx_moe_route_select_check": (C.c_int, [vp, vp]),
        "pmx_moe_set_programmatic_launch": (C.c_int, [C.c_int]),
        "pmx_moe_set_l2_prefetch": (C.c_int, [i32]),
        "pmx_moe_set_weight_prefetch": (C.c_int, [C.c_int]),
        "pmx_moe_set_stamp_buffer": (C.c_int, [vp, sz]),
        "pmx_moe_stamp_slots": (C.c_int, [vp, i32]),
        "pmx_decode_cache_attention_set_kernel": (C.c_int, [i32]),
        "pmx_moe_norm_route_select_workspace_bytes": (sz, [i64, i64, i32, i32, i32]),
        "pmx_moe_norm_route_select": (C.c_int, [vp, vp, vp, f32, vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, i32, i32,
                                                vp, sz, vp]),
        "pmx_moe_select_static": (C.c_int, [vp, vp, vp, vp, vp, vp, i64, i64, i32, i32, i32, vp]),
        "pmx_moe_grouped_linear_workspace_bytes": (sz, [i64, i64, i64, i32, i32, i32, plan_p]),
        "pmx_moe_grouped_linear": (C.c_int, [vp, vp, vp, vp, vp, i64, i64, i64, i32, i32, i32, f32, i32,
                                             plan_p, vp, sz, vp]),
        "pmx_moe_grouped_linear_check": (C.c_int, [vp, C.POINTER(i32 * 4), vp]),
        "pmx_moe_dense_gate_up_covers": (C.c_int, [i64, i64, i64, i32, i32, i32]),
        "pmx_moe_dense_gate_up": (C.c_int, [vp, vp, vp, vp, vp, vp, i64, i64, i64, i32, i32, i32, f32, vp, sz, vp]),
        "pmx_moe_dense_mlp_set_rows": (C.c_int, [i32]),
        "pmx_moe_dense_mlp_covers": (C.c_int, [i64, i64, i64, i32, i32, i32]),
        "pmx_moe_dense_mlp_workspace_bytes": (sz, [i32]),
        "pmx_moe_dense_mlp": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i32, i32, i32, f32, vp, sz, vp]),
        "pmx_moe_dense_mlp_check": (C.c_int, [vp, i32, vp, vp]),
        "pmx_swiglu": (C.c_int, [vp, vp, i64, i64, f32, i32, vp]),
        "pmx_silu": (C.c_int, [vp, vp, vp, i64, i32, vp]),
        "pmx_skip_rms_norm": (C.c_int, [vp, vp, vp, vp, vp, i64, i64, f32, i32, vp]),
        "pmx_moe_reduce": (C.c_int, [vp, vp, vp, vp, i64, i32, i64, i32, vp]),
        "pmx_decode_cache_attention_workspace_bytes": (sz, [i64, i32, i32, i32, i64]),
        "pmx_decode_cache_attention": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, i64, i64, i64, i64, i64,
                                                 i32, vp, sz, vp]),
        "pmx_moe_reduce_allreduce_buffer_bytes": (sz, [i64, i64, i32]),
        "pmx_moe_reduce_allreduce": (C.c_int, [vp, vp, vp, vp, i64, i32, i64, i32, C.POINTER(vp), i32, i32, sz,
                                               i32, i32, i64, vp]),
        "pmx_moe_reduce_allreduce_check": (C.c_int, [vp, C.POINTER(i32 * 4), vp]),
        "pmx_moe_reduce_allreduce_phases": (C.c_int, [vp, C.POINTER(C.c_uint64 * 8), vp]),
        "pmx_moe_reduce_allreduce_emulated": (C.c_int, [C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), i64, i32,
                                                        i64, i32, C.POINTER(vp), i32, sz, i32, i64, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    if lib.pmx_moe_abi_version() != ABI_VERSION:
        raise ImportError("libpmx_moe_b200.so has an unexpected ABI version; rebuild it")
    return lib


lib = _load()


def check(status: int) -> None:
    if status != 0:
        raise PmxError(status, lib.pmx_moe_last_error().decode())


def ptr(t: torch.Tensor | None) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def stream_of(t: torch.Tensor) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


ALLREDUCE_AUTO, ALLREDUCE_PULL, ALLREDUCE_PUSH = 0, 1, 2
ALLREDUCE_FLAG_STAMPS = 1

_barrier_ws: dict = {}


def barrier_workspace(nbytes: int, device, kind: str = "route") -> torch.Tensor:
    """The workspace of the one-launch router + select kernels (kind "route") or of the
    one-launch expert projections (kind "mlp"): its barrier words / counters must be zero
    before the first call and every completed call leaves them zero, so ONE buffer per
    device and kind is allocated (zeroed) on first use and kept.  Calls that share it must
    not overlap on the GPU: callers that drive several streams of one device concurrently
    pass a workspace of their own to the operators instead."""
    dev = torch.device(device)
    key = (dev.index, kind)
    t = _barrier_ws.get(key)
    if t is None or t.numel() < nbytes:
        t = torch.zeros(max(int(nbytes), 64 + 8 * 1024), dtype=torch.uint8, device=dev)
        _barrier_ws[key] = t
    return t


def workspace(nbytes: int, device) -> torch.Tensor:
    # torch's caching allocator hands out 512-byte aligned blocks
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)
