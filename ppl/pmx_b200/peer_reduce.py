"""Host side of the fused moe_reduce + all-reduce over NVLink peer memory
(`pmx_moe_reduce_allreduce`): allocates one symmetric exchange buffer per rank,
maps every peer's buffer into this process and keeps the pointer table.

The weighted combine of MoeReduce (torch_function/MoeReduce.py:23-25) is done
before the sum over ranks that the reference performs on the expanded rows
(torch_function/MoeRowParallelLinear.py:57-58).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ._cabi import lib, check, ptr, stream_of, DTYPE_CODE, ALLREDUCE_AUTO, ALLREDUCE_PULL, ALLREDUCE_PUSH, ALLREDUCE_FLAG_STAMPS

ALGORITHMS = {"auto": ALLREDUCE_AUTO, "pull": ALLREDUCE_PULL, "push": ALLREDUCE_PUSH}

# above this many bytes of [T,N] the one-shot exchange (every rank pulls
# world-1 buffers) loses to NCCL's reduce-scatter + all-gather
ONE_SHOT_LIMIT_BYTES = 4 << 20


class PeerCombine:
    """Exchange buffers of one tensor-parallel group for results of up to
    `max_tokens` x `width` elements of `dtype`."""

    def __init__(self, group, max_tokens: int, width: int, dtype: torch.dtype, device,
                 algorithm: str = "auto", wait_limit_s: float = 0.0, stamps: bool = False):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.algorithm = ALGORITHMS[algorithm]
        self.wait_limit_ns = int(wait_limit_s * 1e9)      # 0: the library's default (1 s)
        self.flags = ALLREDUCE_FLAG_STAMPS if stamps else 0
        self.rank = dist.get_rank(group=group)
        self.world = dist.get_world_size(group=group)
        self.max_tokens, self.width, self.dtype = max_tokens, width, dtype
        self.nbytes = lib.pmx_moe_reduce_allreduce_buffer_bytes(max_tokens, width, DTYPE_CODE[dtype])
        self.buffer = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        assert len(ptrs) == self.world and ptrs[self.rank] == self.buffer.data_ptr()
        self.table = (C.c_void_p * self.world)(*ptrs)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)           # every rank's control block is zero before anyone signals

    def fits(self, tokens: int, width: int, dtype: torch.dtype) -> bool:
        return (dtype == self.dtype and width == self.width and tokens <= self.max_tokens
                and tokens * width * torch.empty((), dtype=dtype).element_size() <= ONE_SHOT_LIMIT_BYTES)

    def combine_allreduce(self, y: torch.Tensor, expert_weights: torch.Tensor,
                          invert_permutation: torch.Tensor, k: int) -> torch.Tensor:
        """y [T*k, N] partial rows of this rank -> [*, N] summed over the group."""
        N = y.shape[-1]
        T = expert_weights.numel() // k
        out = torch.empty(*expert_weights.shape[:-1], N, dtype=y.dtype, device=y.device)
        y2 = y.contiguous()
        w = expert_weights.to(y.dtype).contiguous()
        inv = invert_permutation.contiguous()
        with torch.cuda.device(y.device):
            check(lib.pmx_moe_reduce_allreduce(ptr(y2), ptr(w), ptr(inv), ptr(out), T, k, N, DTYPE_CODE[y.dtype],
                                               self.table, self.rank, self.world, self.nbytes, self.algorithm,
                                               self.flags, self.wait_limit_ns, stream_of(y)))
        return out

    def phases_ns(self):
        """Phase boundaries of CTA 0 in the last call (needs stamps=True), ns after its start."""
        rec = (C.c_uint64 * 8)()
        with torch.cuda.device(self.buffer.device):
            check(lib.pmx_moe_reduce_allreduce_phases(ptr(self.buffer), C.byref(rec), stream_of(self.buffer)))
        t = list(rec)
        if self.algorithm == ALLREDUCE_PULL:
            names = ("combine_done", "epoch_published", "peers_seen", "sum_done")
        else:
            names = ("partials_sent", "owned_sums_published", "all_sums_received")
        return {n: int(t[i + 1]) - int(t[0]) for i, n in enumerate(names)}

    def reset(self) -> None:
        """Zeroes the exchange buffer on every rank and synchronises the group: needed after
        check() reported a wait that ran out (the protocol state is then undefined)."""
        torch.cuda.synchronize(self.buffer.device)
        dist.barrier(group=self.group)
        self.buffer.zero_()
        torch.cuda.synchronize(self.buffer.device)
        dist.barrier(group=self.group)

    def check(self) -> None:
        """Synchronises and raises if a wait on a peer ran out since the last check
        (the record is cleared; call reset() on all ranks before the next exchange)."""
        rec = (C.c_int32 * 4)()
        with torch.cuda.device(self.buffer.device):
            check(lib.pmx_moe_reduce_allreduce_check(ptr(self.buffer), C.byref(rec), stream_of(self.buffer)))
