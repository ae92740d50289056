// Grouped expert GEMM with paired CTAs (tcgen05 cta_group::2), prefill shape.
//
// Two CTAs of a 2-CTA cluster (two SMs) work on one 256-token x N tile:
//   - each CTA loads its own 128 token rows (operand A) and HALF of the weight
//     rows of the tile (operand B) per k-block, so a k-block costs 32 KB of
//     shared memory per CTA instead of 48 KB (six ring stages instead of four)
//     and the weight tile is read from shared memory once per pair;
//   - the leader CTA (cluster rank 0) issues one tcgen05.mma.cta_group::2 with
//     M = 256 per 16-element k-step; the hardware takes A from both CTAs and the
//     two halves of B from both CTAs; each CTA keeps the accumulator of its own
//     128 rows in its own tensor memory;
//   - TMA completions of both CTAs are counted on the LEADER's "full" barrier
//     (the cta_group::2 form of the tensor copy; every CTA fetches its own boxes);
//   - tcgen05.commit.cta_group::2 with a CTA mask releases the ring stage in both
//     CTAs and publishes the accumulator to both CTAs' epilogue warps;
//   - the epilogue warps of both CTAs report a drained accumulator buffer to the
//     leader's barrier (the peer arrives through the cluster address).
// Roles per CTA as in the single-CTA kernel: warp 0 TMA producer, warp 1 tensor
// memory owner (and, in the leader, the MMA issuer), warps 2-5 epilogue.
// With SwiGLU the leader's half of B holds the gate rows and the peer's half the
// up rows, so accumulator columns [0,ft) are gate and [ft,2ft) up, as in the
// single-CTA kernel.  All waits are bounded (2 s) as there.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <type_traits>

#include "common.cuh"

namespace pmx {
namespace {

#include "tcgen05_common.cuh"

constexpr uint32_t kLeaderMask = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared::cluster address

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* holder, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(holder)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// TMA load whose completion is counted on the leader CTA's barrier
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar) & kLeaderMask), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive (once all MMAs issued so far are done) on the barrier at this offset in both CTAs
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(static_cast<uint16_t>(3))
      : "memory");
}
// arrive on the leader CTA's copy of a barrier
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & kLeaderMask)
               : "memory");
}

template <typename T, bool SWIGLU>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
grouped_gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x,
                            const __grid_constant__ CUtensorMap map_w, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int ft = p.tile_feat;
  const int wrows = SWIGLU ? 2 * ft : ft;       // weight rows of the pair's tile = MMA N
  const int my_wrows = wrows / 2;               // ... of which this CTA loads half
  const uint32_t tok_bytes = 128 * 128, w_bytes = my_wrows * 128;
  const uint32_t stage_bytes = tok_bytes + w_bytes;
  Shared* sh = reinterpret_cast<Shared*>(smem + (size_t)p.stages * stage_bytes);
  int* s_off = reinterpret_cast<int*>(sh + 1);
  int* s_prefix = s_off + (p.E + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  // set-up that touches nothing another kernel writes: under programmatic dependent
  // launch it overlaps the tail of the kernel in front
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; ++i) {
      mbar_init(&sh->full[i], 1);    // used in the leader only: its producer's expect_tx arrival
      mbar_init(&sh->empty[i], 1);   // one commit from the leader's MMA thread
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh->acc_full[i], 1);
      mbar_init(&sh->acc_empty[i], 8);  // used in the leader only: 4 epilogue warps of each CTA
    }
    sh->abort = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_x);
    prefetch_tensormap(&map_w);
  }
  if (warp == 1) {
    tmem_alloc2(&sh->tmem_base, kTmemCols);
    tmem_relinquish2();
  }
  pdl_wait();
  if (blockIdx.x == 0 && threadIdx.x < 4) p.status[threadIdx.x] = 0;
  for (int e = threadIdx.x; e <= p.E; e += blockDim.x) {
    long long o = offset_at(p.off, e, p.M);
    s_off[e] = (int)(o < 0 ? 0 : (o > p.M ? p.M : o));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < p.E; ++e) {
      if (s_off[e + 1] < s_off[e]) s_off[e + 1] = s_off[e];
      s_prefix[e] = acc;
      const int rows = s_off[e + 1] - s_off[e];
      acc += ((rows + 255) / 256) * p.feat_tiles;   // the pair's token tile is 256 rows
    }
    s_prefix[p.E] = acc;
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();   // both CTAs' barriers are initialised before any remote arrival
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  const int total_items = s_prefix[p.E];
  const uint32_t smem_base = smem_u32(smem);
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ========================= TMA producer (both CTAs) =====================
    if (lane == 0) {
      int stage = 0, e = 0;
      uint32_t phase = 0;
      Item it;
      bool ok = true;
      for (int item = pair; item < total_items && ok; item += pairs) {
        decode_item(item, e, s_off, s_prefix, p, it);
        // weight rows this CTA fetches: SwiGLU -> leader the gate rows, peer the up rows;
        // otherwise the two halves of the feature tile
        const int wrow = it.e * p.w_pitch + it.f0 + (SWIGLU ? (int)rank * (p.N / 2) : (int)rank * my_wrows);
        const int row0 = it.row0 + (int)rank * 128;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          ok = wait_barrier(&sh->empty[stage], phase ^ 1u, sh, p.status, 0, item);
          if (!ok) break;
          if (leader) mbar_expect_tx(&sh->full[stage], 2 * stage_bytes);
          const uint32_t dst = smem_base + stage * stage_bytes;
          tma_load_2d_pair(dst, &map_x, &sh->full[stage], kb * kBlockK, row0);
          tma_load_2d_pair(dst + tok_bytes, &map_w, &sh->full[stage], kb * kBlockK, wrow);
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 1000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ========================= MMA issuer (leader only) =====================
    if (leader && lane == 0) {
      const uint32_t idesc = make_idesc<T>(256, wrows);
      int stage = 0, acc = 0, e = 0;
      uint32_t phase = 0, acc_phase = 0;
      Item it;
      bool ok = true;
      for (int item = pair; item < total_items && ok; item += pairs) {
        decode_item(item, e, s_off, s_prefix, p, it);
        ok = wait_barrier(&sh->acc_empty[acc], acc_phase ^ 1u, sh, p.status, 1, item);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kAccStride;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          ok = wait_barrier(&sh->full[stage], phase, sh, p.status, 2, item);
          if (!ok) break;
          tc_fence_after();
          const uint32_t tok_addr = smem_base + stage * stage_bytes;
          const uint32_t w_addr = tok_addr + tok_bytes;
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
            const uint32_t koff = kk * kUmmaK * 2;
            umma_f16_pair(d_tmem, smem_desc_sw128(tok_addr + koff), smem_desc_sw128(w_addr + koff), idesc,
                          (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_pair(&sh->empty[stage]);
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit_pair(&sh->acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ========================= epilogue (both CTAs) ==========================
    const int q = warp & 3;
    int acc = 0, e = 0;
    uint32_t acc_phase = 0;
    Item it;
    bool ok = true;
    T* y = reinterpret_cast<T*>(p.y);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    for (int item = pair; item < total_items; item += pairs) {
      decode_item(item, e, s_off, s_prefix, p, it);
      ok = wait_barrier(&sh->acc_full[acc], acc_phase, sh, p.status, 3, item);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * kAccStride + (static_cast<uint32_t>(q * 32) << 16);
      const int row = it.row0 + (int)rank * 128 + q * 32 + lane;
      const bool row_ok = row < it.row_end;
      const T* be = bias ? bias + (int64_t)it.e * p.w_pitch : nullptr;
      // 16 accumulator columns of this thread's row: bias, SwiGLU, cast, store
      auto emit = [&](int col, float (&g)[16], float (&u)[16]) {
        if (col >= p.n_out || !row_ok) return;
        if (be) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (col + i < p.n_out) {
              g[i] += Elem<T>::to_f(be[col + i]);
              if (SWIGLU) u[i] += Elem<T>::to_f(be[p.n_out + col + i]);
            }
        }
        if (SWIGLU) {
#pragma unroll
          for (int i = 0; i < 16; ++i) g[i] = swiglu_f(g[i], u[i], p.beta);
        }
        T* dst = y + (int64_t)row * p.n_out + col;
        if (col + 16 <= p.n_out) {
          store16<T>(dst, g);
        } else {
          for (int i = 0; i < 16 && col + i < p.n_out; ++i) dst[i] = Elem<T>::from_f(g[i]);
        }
      };
      // 32 columns per round: both halves' tensor-memory loads are in flight before the wait
      for (int c = 0; c < ft; c += 32) {
        const bool two = c + 32 <= ft;
        float g0[16], g1[16], u0[16], u1[16];
        __syncwarp();
        tmem_ld16(taddr + c, g0);
        if (two) tmem_ld16(taddr + c + 16, g1);
        if (SWIGLU) {
          tmem_ld16(taddr + ft + c, u0);
          if (two) tmem_ld16(taddr + ft + c + 16, u1);
        }
        tmem_wait_ld();
        emit(it.f0 + c, g0, u0);
        if (two) emit(it.f0 + c + 16, g1, u1);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&sh->acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---- common exit: nobody leaves while the pair may still touch its memory ------
  tc_fence_before();
  __syncthreads();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, kTmemCols);
  }
}

template <typename T, bool SWIGLU>
int launch_pair_inst(const CUtensorMap& mx, const CUtensorMap& mw, const Params& p, int grid, size_t smem,
                     cudaStream_t s) {
  auto kern = grouped_gemm_tc_pair_kernel<T, SWIGLU>;
  PMX_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  void* args[] = {(void*)&mx, (void*)&mw, (void*)&p};
  // the cluster shape is part of the kernel (__cluster_dims__)
  return launch_pdl((const void*)kern, dim3(grid), dim3(kThreads), smem, s, args);
}

}  // namespace

// Plan for the paired kernel; false if the shape is outside what it covers.
bool plan_gemm_tc_pair(int64_t M, int64_t N, int64_t K, int E, int dtype, int epilogue,
                       const pmx_gemm_plan* user, TcPlan* plan) {
  const bool swiglu = epilogue == PMX_EPILOGUE_SWIGLU;
  const int64_t n_out = swiglu ? N / 2 : N;
  if (dtype != PMX_DTYPE_F16 && dtype != PMX_DTYPE_BF16) return false;
  if (K % 8 || n_out % 8 || K < 8 || E > kMaxExperts) return false;
  if (M >= (1ll << 31) || (int64_t)E * N >= (1ll << 31) || M * n_out >= (1ll << 40)) return false;
  TcPlan pl{};
  pl.kernel = PMX_GEMM_TC_TOKENS_M_PAIRED;
  pl.tile_tok = 256;
  const int ft_max = swiglu ? 128 : 256;
  int ft = user && user->tile_feat ? user->tile_feat : ft_max;
  while (!(user && user->tile_feat) && ft > 32 && ft / 2 >= n_out) ft /= 2;
  if (ft % 32 || ft < 32 || ft > ft_max) return false;   // each CTA's half must be a multiple of 16 rows
  pl.tile_feat = ft;
  pl.split_k = 1;
  pl.stream_k = 0;
  const int wrows = swiglu ? 2 * ft : ft;
  const size_t stage = (size_t)(128 + wrows / 2) * 128;
  const size_t fixed = 1024 + sizeof(Shared) + 2 * (size_t)(E + 1) * sizeof(int);
  int st = (int)((227 * 1024 - fixed) / stage);
  if (st > 8) st = 8;
  if (user && user->stages) st = user->stages < st ? user->stages : st;
  if (st < 2) return false;
  pl.stages = st;
  const int sms = sm_count();
  int ctas = user && user->max_ctas ? user->max_ctas : sms;
  ctas &= ~1;
  if (ctas < 2) return false;
  pl.max_ctas = ctas;
  pl.cta_cap = ctas;
  pl.full_rounds = 0;
  *plan = pl;
  return true;
}

int launch_gemm_tc_pair(const void* x, const int64_t* off, const void* w, const void* bias, void* y,
                        int64_t M, int64_t N, int64_t K, int E, int dtype, int epilogue, float beta,
                        const TcPlan& plan, void* ws, size_t ws_bytes, cudaStream_t s) {
  const bool swiglu = epilogue == PMX_EPILOGUE_SWIGLU;
  const int64_t n_out = swiglu ? N / 2 : N;
  if (!aligned16(x) || !aligned16(w) || !aligned16(y))
    return fail(PMX_ERR_ALIGNMENT, "grouped_linear: x, w and y must be 16-byte aligned");
  if (!ws || ws_bytes < kStatusBytes) return fail(PMX_ERR_WORKSPACE, "grouped_linear: workspace of %zu bytes needed, %zu given", kStatusBytes, ws_bytes);
  const int wrows = swiglu ? 2 * plan.tile_feat : plan.tile_feat;
  CUtensorMap mx, mw;
  int st = make_map(&mx, x, (uint64_t)M, (uint64_t)K, 128u, dtype);
  if (st != PMX_OK) return st;
  st = make_map(&mw, w, (uint64_t)(E - 1) * (uint64_t)(plan.w_pitch > 0 ? plan.w_pitch : N) + (uint64_t)N, (uint64_t)K, (uint32_t)(wrows / 2), dtype);
  if (st != PMX_OK) return st;
  Params p{};
  p.off = off;
  p.bias = bias;
  p.status = reinterpret_cast<int*>(ws);
  p.y = y;
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.E = E;
  p.w_pitch = plan.w_pitch > 0 ? plan.w_pitch : (int)N;
  p.n_out = (int)n_out;
  p.tile_tok = 256;
  p.tile_feat = plan.tile_feat;
  p.feat_tiles = (int)ceil_div(n_out, plan.tile_feat);
  p.kblocks = (int)ceil_div(K, kBlockK);
  p.split_k = 1;
  p.kb_per_split = p.kblocks;
  p.stages = plan.stages;
  p.beta = beta;
  p.cta_cap = plan.max_ctas;
  const size_t smem = 1024 + (size_t)(128 + wrows / 2) * 128 * plan.stages + sizeof(Shared) + 2 * (size_t)(E + 1) * sizeof(int);
  const bool bf = dtype == PMX_DTYPE_BF16;
  if (swiglu) return bf ? launch_pair_inst<__nv_bfloat16, true>(mx, mw, p, plan.max_ctas, smem, s)
                        : launch_pair_inst<__half, true>(mx, mw, p, plan.max_ctas, smem, s);
  return bf ? launch_pair_inst<__nv_bfloat16, false>(mx, mw, p, plan.max_ctas, smem, s)
            : launch_pair_inst<__half, false>(mx, mw, p, plan.max_ctas, smem, s);
}

}  // namespace pmx
