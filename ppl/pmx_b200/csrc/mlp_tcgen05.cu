// Decode-size expert feed-forward in ONE launch on the 5th-generation tensor cores:
//   h[r,:] = SwiGLU(x[t,:] . wu[e]^T)      for every token t and every expert e it chose,
//   y[r,:] = h[r,:] . w2[e]^T              r = the row of (t,e) in the expert-sorted order,
// i.e. moe_column_parallel_linear + swiglu + moe_row_parallel_linear of the reference
// (MoeColumnParallelLinear.py:58-69, SwiGLU.py:15-16, MoeRowParallelLinear.py:44-55) for a
// batch of at most 64 tokens, without the launch boundary between the two projections.
//
// A thin tensor-parallel shard streams its weights in a few tens of microseconds, so the
// fixed cost of a launch (set-up, first-load latency, the drain of the last tiles) is a
// large part of each projection.  Here both projections are work items of one persistent
// grid (one CTA per SM, weight rows on MMA-M, all T tokens on MMA-N as in the dense
// gate/up kernel):
//   phase 1  items (expert, 128 gate + 128 up rows of wu), K = hidden;
//   phase 2  items (expert, 256 rows of w2),               K = this shard's intermediate dim.
// A CTA works through its phase-1 items, then its phase-2 items, with ONE ring of
// shared-memory stages: the producer keeps requesting weight tiles (they depend on
// nothing) and adds the token-side tile of a stage (x, or the rows of h) separately, so
// the w2 stream is already in flight while the last gate/up tiles are finished elsewhere.
// The rows of h for expert e are complete when all its gate/up tiles have counted
// themselves in done[e] (4 epilogue warps per tile); the producer polls that counter
// before it requests the first h tile of a phase-2 item of e.  Phase-1 items wait for
// nothing, and a CTA finishes them before its phase-2 items, so the waits cannot form a
// cycle; the grid is at most one CTA per SM, so all CTAs are resident.  The last CTA to
// leave clears the counters: they are zero before the first launch and after every one.
//
// Roles, barriers, bounded waits and the abort path are those of grouped_gemm_tc_kernel.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <atomic>
#include <type_traits>

#include "common.cuh"

namespace pmx {
namespace {

#include "tcgen05_common.cuh"

constexpr int kMlpMaxTokens = 128;  // tokens on MMA-N: two accumulator halves of that many columns fill a 256-column buffer

struct MlpParams {
  const int64_t* off;   // [E+1]
  const int64_t* inv;   // [T,k]
  void* h;              // [T*k, I]
  void* y;              // [T*k, H]
  int* status;          // 4 ints: code, role, item, aux
  unsigned int* done;   // [E] gate/up epilogue warps finished per expert; [E] = CTAs that have left
  int T, E, k;
  int I, H;             // this shard's intermediate features, hidden features
  int tile_tok;         // tokens on MMA-N: T rounded up to 16
  int r1;               // phase 1: gate rows (= up rows) per work item, a multiple of 8, <= 128
  int stages1, stages2; // ring depth in phase 1 (stages of tile_tok + 2 r1 rows) and phase 2 (tile_tok + 256 rows)
  int ring_bytes;       // shared memory the ring may use (the larger of the two shapes, plus what the
                        // 128-row MMA operand of a shorter tile reads behind the last stage)
  int f1, f2;           // work items per expert: ceil(I/r1), ceil(H/256)
  int kb1, kb2;         // k-blocks per item: ceil(H/64), ceil(I/64)
  int g1, g2;           // CTAs that take phase-1 / phase-2 items
  unsigned long long* stamps;   // diagnostic: [cta][8] %globaltimer values, or null
  int l2_ahead;         // weight tiles are requested into L2 this many k-blocks in front of the ring
  float beta;
};

// The work of one CTA: items [a1,b1) of phase 1, then [a2,b2) of phase 2, each a run of k-blocks.
struct Cursor {
  int phase;            // 1, 2; 3 = finished
  int item, end, kb;
  int a2, b2;
  int e, f;             // expert and tile of the current item (divisions once per item, not per k-block)
  __device__ __forceinline__ void locate(const MlpParams& p) {
    if (phase == 3) return;
    const int per = phase == 1 ? p.f1 : p.f2;
    e = item / per;
    f = item - e * per;
  }
  __device__ __forceinline__ void init(const MlpParams& p) {
    const int c = (int)blockIdx.x;
    const int n1 = p.E * p.f1, n2 = p.E * p.f2;
    int a1 = 0, b1 = 0;
    a2 = b2 = 0;
    if (c < p.g1) {
      a1 = (int)((long long)c * n1 / p.g1);
      b1 = (int)((long long)(c + 1) * n1 / p.g1);
    }
    if (c < p.g2) {
      a2 = (int)((long long)c * n2 / p.g2);
      b2 = (int)((long long)(c + 1) * n2 / p.g2);
    }
    kb = 0;
    phase = 1; item = a1; end = b1;
    if (item >= end) { phase = 2; item = a2; end = b2; }
    if (item >= end) phase = 3;
    e = f = 0;
    locate(p);
  }
  __device__ __forceinline__ void next_item(const MlpParams& p) {
    kb = 0;
    if (++item >= end) {
      if (phase == 1) {
        phase = 2; item = a2; end = b2;
        if (item >= end) phase = 3;
      } else {
        phase = 3;
      }
    }
    locate(p);
  }
  __device__ __forceinline__ void next_kblock(const MlpParams& p) {
    if (++kb == (phase == 1 ? p.kb1 : p.kb2)) next_item(p);
  }
};

__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// orders this thread's earlier generic-proxy accesses of global memory against later
// accesses through the async proxy (TMA): h is written with plain stores and read by TMA
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
expert_mlp_decode_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_wu,
                         const __grid_constant__ CUtensorMap map_h, const __grid_constant__ CUtensorMap map_w2,
                         const MlpParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tt = p.tile_tok;
  // The ring has one shape per phase (same shared memory, barriers 0.. for phase 1 and
  // kBar2.. for phase 2): phase 1 stages hold the token tile and r1 gate + r1 up rows, phase 2
  // stages the token tile and 256 rows of w2.  r1 < 128 is how 128 (or more) CTAs get a whole
  // item each when the shard has fewer than 128 tiles of 128 rows -- more CTAs streaming and a
  // deeper ring mean more bytes in flight, which is what the rate of a thin shard depends on.
  constexpr int kBar2 = 8;
  const uint32_t tok_bytes = tt * 128;
  const uint32_t half1 = p.r1 * 128;                 // bytes of the gate (or up) rows of a phase-1 stage
  const uint32_t sb1 = tok_bytes + 2 * half1, sb2 = tok_bytes + 256 * 128;
  Shared* sh = reinterpret_cast<Shared*>(smem + (size_t)p.ring_bytes);
  int* s_rowmap = reinterpret_cast<int*>(sh + 1);    // [4 warps][128]: output row of every token for the current expert
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- set-up: nothing here touches memory another kernel writes ---------------
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    stamp(p.stamps, 0);
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(&sh->full[i], 1);
      mbar_init(&sh->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh->acc_full[i], 1);
      mbar_init(&sh->acc_empty[i], 4);
    }
    sh->abort = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_x);
    prefetch_tensormap(&map_wu);
    prefetch_tensormap(&map_h);
    prefetch_tensormap(&map_w2);
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  const uint32_t smem_base = smem_u32(smem);
  if (threadIdx.x == 0) stamp(p.stamps, 1);
  const unsigned int tiles_done = 4u * (unsigned int)p.f1;   // value of done[e] once h of expert e is complete

  if (warp == 0) {
    // ========================= TMA producer =================================
    // Two cursors over the same sequence of k-blocks: `w` requests weight tiles as soon as a
    // stage is free, `t` follows with the token-side tile of the same stage (at most `stages`
    // behind) once what it reads exists.
    if (lane == 0) {
      Cursor w, t, pf;
      w.init(p);
      t.init(p);
      pf.init(p);
      // L2 prefetch cursor, p.l2_ahead k-blocks in front of `w` (the ring itself covers the first `stages`)
      auto prefetch_step = [&](bool issue) {
        if (pf.phase == 3) return;
        if (issue) {
          if (pf.phase == 1) {
            const int row = pf.e * 2 * p.I + pf.f * p.r1;
            tma_prefetch_l2_2d(&map_wu, pf.kb * kBlockK, row);
            tma_prefetch_l2_2d(&map_wu, pf.kb * kBlockK, row + p.I);
          } else {
            const int row = pf.e * p.H + pf.f * 256;
            tma_prefetch_l2_2d(&map_w2, pf.kb * kBlockK, row);
            tma_prefetch_l2_2d(&map_w2, pf.kb * kBlockK, row + 128);
          }
        }
        pf.next_kblock(p);
      };
      if (p.l2_ahead > 0)
        for (int i = 0; i < p.stages1 + p.l2_ahead; ++i) prefetch_step(i >= p.stages1);
      int w_stage = 0, t_stage = 0, pending = 0;
      uint32_t w_phase = 0;
      int ring = w.phase == 2 ? 2 : 1;            // the shape the ring has now
      int nst = ring == 1 ? p.stages1 : p.stages2, bar0 = ring == 1 ? 0 : kBar2;
      uint32_t sb = ring == 1 ? sb1 : sb2;
      int ready_e = -1;          // expert whose rows of h are known to be complete
      int ready_row = 0;         // ... and its first row in h
      bool routed = false;       // pdl_wait() done: expert_offset may be read
      bool ok = true;
      while (ok && t.phase != 3) {
        while (pending > 0) {
          const int e = t.e;
          if (t.phase == 2) {
            if (e != ready_e) {
              const bool must = pending == nst || w.phase == 3;   // nothing else to request
              if (!routed) {
                // The counters belong to this launch only once every kernel in front has
                // finished (an earlier launch of this kernel clears them as it leaves), and
                // expert_offset is the routing kernel's: wait for them -- but not while
                // there are weight tiles to request.
                if (!must) break;
                pdl_wait();
                routed = true;
              }
              bool ready = ld_acquire_gpu_u32(p.done + e) >= tiles_done;
              if (!ready && must) {
                // nothing else to request: wait (bounded) for the gate/up tiles of expert e
                const unsigned long long t0 = global_ns();
                for (unsigned int spin = 1;; ++spin) {
                  if (ld_acquire_gpu_u32(p.done + e) >= tiles_done) { ready = true; break; }
                  if ((spin & 15u) == 0u) {
                    if (sh->abort) break;
                    if (global_ns() - t0 > kWaitLimitNs) {
                      sh->abort = 1;
                      if (atomicExch(p.status, 1) != 1) { p.status[1] = 5; p.status[2] = t.item; p.status[3] = (int)blockIdx.x; }
                      break;
                    }
                  }
                }
                if (!ready) { ok = false; break; }
              }
              if (!ready) break;
              fence_proxy_async_global();
              ready_e = e;
              long long r0 = p.off[e];      // first row of expert e in h (once per expert, not per k-block)
              ready_row = (int)(r0 < 0 ? 0 : (r0 > (long long)p.T * p.k ? (long long)p.T * p.k : r0));
            }
          }
          const uint32_t dst = smem_base + t_stage * sb;
          uint64_t* bar = &sh->full[bar0 + t_stage];
          mbar_expect_tx(bar, tok_bytes);
          if (t.phase == 1) {
            tma_load_2d(dst, &map_x, bar, t.kb * kBlockK, 0);
          } else {
            tma_load_2d(dst, &map_h, bar, t.kb * kBlockK, ready_row);
          }
          t.next_kblock(p);
          if (++t_stage == nst) t_stage = 0;
          --pending;
        }
        if (!ok) break;
        if (w.phase != 3 && pending < nst) {
          if (w.phase != ring) {
            // Phase 1 is requested completely (and, x being there from the start, `t` has caught
            // up: pending is 0).  The ring takes its phase-2 shape once the MMAs have read every
            // phase-1 stage: stage s was last filled in this pass over the ring if s < w_stage,
            // in the pass before otherwise.
            for (int s = 0; s < p.stages1 && ok; ++s)
              ok = wait_barrier(&sh->empty[s], s < w_stage ? w_phase : w_phase ^ 1u, sh, p.status, 0, w.item);
            if (!ok) break;
            ring = 2; nst = p.stages2; bar0 = kBar2; sb = sb2;
            w_stage = t_stage = 0;
            w_phase = 0;
          }
          ok = wait_barrier(&sh->empty[bar0 + w_stage], w_phase ^ 1u, sh, p.status, 0, w.item);
          if (!ok) break;
          const uint32_t dst = smem_base + w_stage * sb + tok_bytes;
          uint64_t* bar = &sh->full[bar0 + w_stage];
          if (p.l2_ahead > 0) prefetch_step(true);
          if (w.phase == 1) {
            const int row = w.e * 2 * p.I + w.f * p.r1;
            mbar_expect_tx_only(bar, 2 * half1);
            tma_load_2d(dst, &map_wu, bar, w.kb * kBlockK, row);
            tma_load_2d(dst + half1, &map_wu, bar, w.kb * kBlockK, row + p.I);
          } else {
            const int row = w.e * p.H + w.f * 256;
            mbar_expect_tx_only(bar, 256 * 128);
            tma_load_2d(dst, &map_w2, bar, w.kb * kBlockK, row);
            tma_load_2d(dst + 128 * 128, &map_w2, bar, w.kb * kBlockK, row + 128);
          }
          w.next_kblock(p);
          if (++w_stage == nst) { w_stage = 0; w_phase ^= 1u; }
          ++pending;
        }
      }
      if (!ok) {
        // leave time for copies already in flight to land before the CTA exits
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 1000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ========================= MMA issuer ===================================
    if (lane == 0) {
      const uint32_t idesc = make_idesc<T>(128, tt);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      Cursor c;
      c.init(p);
      bool ok = true;
      bool first_tile = true, first_down = true;
      int ring = c.phase == 2 ? 2 : 1;
      while (ok && c.phase != 3) {
        if (c.phase != ring) { ring = 2; stage = 0; phase = 0; }     // the ring's phase-2 shape and barriers
        const int nst = ring == 1 ? p.stages1 : p.stages2, bar0 = ring == 1 ? 0 : kBar2;
        const uint32_t sb = ring == 1 ? sb1 : sb2, second = ring == 1 ? half1 : 128u * 128u;
        ok = wait_barrier(&sh->acc_empty[acc], acc_phase ^ 1u, sh, p.status, 1, c.item);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kAccStride;
        const int nkb = c.phase == 1 ? p.kb1 : p.kb2;
        for (int kb = 0; kb < nkb; ++kb) {
          ok = wait_barrier(&sh->full[bar0 + stage], phase, sh, p.status, 2, c.item);
          if (!ok) break;
          if (p.stamps) {
            if (first_tile) { stamp(p.stamps, 2); first_tile = false; }
            if (c.phase == 2 && kb == 0 && first_down) { stamp(p.stamps, 7); first_down = false; }   // first tile of h arrived
          }
          tc_fence_after();
          const uint32_t tok_addr = smem_base + stage * sb;
          const uint32_t w_addr = tok_addr + tok_bytes;
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
            const uint32_t koff = kk * kUmmaK * 2;  // bytes inside the 128-byte row
            const uint32_t accum = (kb > 0 || kk > 0) ? 1u : 0u;
            const uint64_t bdesc = smem_desc_sw128(tok_addr + koff);
            umma_f16(d_tmem, smem_desc_sw128(w_addr + koff), bdesc, idesc, accum);
            umma_f16(d_tmem + tt, smem_desc_sw128(w_addr + second + koff), bdesc, idesc, accum);
          }
          umma_commit(&sh->empty[bar0 + stage]);
          if (++stage == nst) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&sh->acc_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        c.next_item(p);
      }
      stamp(p.stamps, 3);
    }
  } else {
    // ========================= epilogue (warps 2..5) ========================
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    Cursor c;
    c.init(p);
    T* h = reinterpret_cast<T*>(p.h);
    T* y = reinterpret_cast<T*>(p.y);
    int map_expert = -1;
    pdl_wait();   // the routing (invert_permutation, expert_offset) is complete from here on
    if (blockIdx.x == 0 && warp == 2 && lane < 4) p.status[lane] = 0;
    if (warp == 2 && lane == 0) stamp(p.stamps, 4);
    while (c.phase != 3) {
      const bool gate_up = c.phase == 1;
      const int e = c.e, f = c.f;
      const long long lo = p.off[e], hi = p.off[e + 1];
      if (gate_up && e != map_expert) {
        // which row of the expert-sorted order holds token t for this expert (-1: not routed here)
        __syncwarp();
        for (int t = lane; t < 128; t += 32) {
          int r = -1;
          if (t < p.T) {
            for (int j = 0; j < p.k; ++j) {
              const long long v = p.inv[(long long)t * p.k + j];
              if (v >= lo && v < hi) r = (int)v;
            }
          }
          s_rowmap[q * 128 + t] = r;
        }
        __syncwarp();
        map_expert = e;
      }
      bool ok = wait_barrier(&sh->acc_full[acc], acc_phase, sh, p.status, 3, c.item);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * kAccStride + (static_cast<uint32_t>(q * 32) << 16);
      // Up to 32 columns of both halves per round: their tensor-memory loads are all in flight
      // before the one wait (a tcgen05.ld round trip costs several hundred ns).  Not more: with
      // all 64 columns in registers the kernel needs > 200 registers per thread, and two of its
      // warps no longer fit beside two warps of the routing kernel in an SM sub-partition's
      // register file -- the CTAs on the router's SMs then start 9 us late.
      const int rows = (int)(hi - lo < 0 ? 0 : (hi - lo > tt ? tt : hi - lo));
      const int ncol = gate_up ? (p.T < tt ? p.T : tt) : rows;     // accumulator columns that matter
      const int colg = f * p.r1 + q * 32 + lane;                   // phase 1: feature of h this thread owns
      const bool colg_ok = q * 32 + lane < p.r1 && colg < p.I;
      const int col0 = f * 256 + q * 32 + lane, col1 = col0 + 128; // phase 2: features of y this thread owns
      for (int c0 = 0; c0 < ncol; c0 += 32) {
        float a[2][16], b[2][16];
        __syncwarp();
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          if (c0 + ch * 16 < ncol) {
            tmem_ld16(taddr + c0 + ch * 16, a[ch]);
            tmem_ld16(taddr + tt + c0 + ch * 16, b[ch]);
          }
        }
        tmem_wait_ld();
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          if (c0 + ch * 16 < ncol) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int cc = c0 + ch * 16 + i;
              if (gate_up) {
                const int row = s_rowmap[q * 128 + cc];
                if (row >= 0 && colg_ok)
                  h[(int64_t)row * p.I + colg] = Elem<T>::from_f(swiglu_f(a[ch][i], b[ch][i], p.beta));
              } else if (cc < rows) {
                T* dst = y + (int64_t)(lo + cc) * p.H;
                if (col0 < p.H) dst[col0] = Elem<T>::from_f(a[ch][i]);
                if (col1 < p.H) dst[col1] = Elem<T>::from_f(b[ch][i]);
              }
            }
          }
        }
      }
      if (gate_up) {
        // this warp's part of the tile is in global memory: count it for the down projection
        __threadfence();
        fence_proxy_async_global();
        __syncwarp();
        if (lane == 0) atomicAdd(p.done + e, 1u);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      c.next_item(p);
    }
    if (warp == 2 && lane == 0) stamp(p.stamps, 5);
  }

  // ---- common exit ------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) stamp(p.stamps, 6);
  if (threadIdx.x == 64) {
    // the last CTA to leave puts the counters back to zero for the next launch
    __threadfence();
    if (atomicAdd(p.done + p.E, 1u) == gridDim.x - 1) {
      for (int e = 0; e <= p.E; ++e) p.done[e] = 0u;
    }
  }
}

constexpr size_t kRowMapBytes = 4 * 128 * sizeof(int);

// CTAs that take the n items of a phase: the smallest grid that needs no more rounds than
// `cap` CTAs would, so that every round is full
int full_round_grid(int n, int cap) {
  if (n <= 0) return 0;
  const int rounds = (n + cap - 1) / cap;
  return (n + rounds - 1) / rounds;
}

std::atomic<int> g_mlp_rows{0};

}  // namespace

int dense_mlp_set_rows(int rows) {
  return g_mlp_rows.exchange(rows >= 64 && rows <= 128 && rows % 8 == 0 ? rows : 0, std::memory_order_relaxed);
}

bool dense_mlp_covers(int64_t T, int64_t N, int64_t H, int E, int k, int dtype) {
  return T >= 1 && T <= kMlpMaxTokens && E >= 1 && E <= kMaxExperts && k >= 1 && k <= E && N >= 16 && N % 16 == 0 &&
         H >= 8 && H % 8 == 0 && (dtype == PMX_DTYPE_F16 || dtype == PMX_DTYPE_BF16) &&
         (int64_t)E * N < (1ll << 31) && (int64_t)E * H < (1ll << 31);
}

size_t dense_mlp_workspace_bytes(int E) { return kStatusBytes + (size_t)(E + 1) * sizeof(unsigned int); }

int launch_dense_mlp(const void* x, const int64_t* inv, const int64_t* off, const void* wu, const void* w2, void* h,
                     void* y, int64_t T, int64_t N, int64_t H, int E, int k, int dtype, float beta, void* ws,
                     size_t ws_bytes, cudaStream_t s) {
  if (!x || !inv || !off || !wu || !w2 || !h || !y) return fail(PMX_ERR_INVALID_ARGUMENT, "dense_mlp: null pointer");
  if (!dense_mlp_covers(T, N, H, E, k, dtype))
    return fail(PMX_ERR_UNSUPPORTED, "dense_mlp: covers 1..%d tokens, float16 / bfloat16, N a multiple of 16 and H of 8 (T=%lld N=%lld H=%lld)", kMlpMaxTokens, (long long)T, (long long)N, (long long)H);
  if (!aligned16(x) || !aligned16(wu) || !aligned16(w2) || !aligned16(h) || !aligned16(y))
    return fail(PMX_ERR_ALIGNMENT, "dense_mlp: x, wu, w2, h and y must be 16-byte aligned");
  if (!ws || ws_bytes < dense_mlp_workspace_bytes(E) || !aligned16(ws))
    return fail(PMX_ERR_WORKSPACE, "dense_mlp: a 16-byte aligned workspace of %zu bytes is needed", dense_mlp_workspace_bytes(E));
  const int64_t I = N / 2;
  MlpParams p{};
  p.off = off;
  p.inv = inv;
  p.h = h;
  p.y = y;
  p.status = reinterpret_cast<int*>(ws);
  p.done = reinterpret_cast<unsigned int*>(reinterpret_cast<uint8_t*>(ws) + kStatusBytes);
  p.T = (int)T; p.E = E; p.k = k;
  p.I = (int)I; p.H = (int)H;
  p.tile_tok = (int)(ceil_div(T, 16) * 16);
  p.f2 = (int)ceil_div(H, 256);
  p.kb1 = (int)ceil_div(H, kBlockK);
  p.kb2 = (int)ceil_div(I, kBlockK);
  p.beta = beta;
  p.l2_ahead = default_l2_prefetch();
  p.stamps = next_stamp_slot(4);
  const int sms = sm_count();
  const size_t tok = (size_t)p.tile_tok * 128;
  const size_t fixed = 1024 + sizeof(Shared) + kRowMapBytes;
  // 4 KB of every SM's shared memory stay free, so that a CTA of the routing kernel (which asks
  // for the same carve-out) and a CTA of this one fit on an SM together
  const size_t budget = 223 * 1024 - fixed;
  // Phase 1: rows per item.  The rate of a thin shard's weight stream grows with the bytes in
  // flight (CTAs x ring depth x weight bytes per stage) until about 26 MB; a CTA's time is
  // its rows x k-blocks.  Model: time ~ rounds x rows x CTAs / min(in flight, 26 MB).
  double best = 0.0;
  p.r1 = 0;
  const int forced = g_mlp_rows.load(std::memory_order_relaxed);
  for (int r = 128; r >= 64; r -= 8) {
    if (forced && r != forced) continue;
    const int64_t items = (int64_t)E * ceil_div(I, r);
    const int64_t rounds = ceil_div(items, sms);
    const int64_t ctas = ceil_div(items, rounds);
    const size_t stage = tok + 2 * (size_t)r * 128;
    const size_t pad = (size_t)(128 - r) * 128;            // what the 128-row operand reads behind a short tile
    if (budget < pad + 2 * stage) continue;
    int st1 = (int)((budget - pad) / stage);
    if (st1 > 8) st1 = 8;
    const double flight = (double)ctas * st1 * 2.0 * r * 128.0;
    const double t = (double)rounds * r * (double)ctas / (flight < 26e6 ? flight : 26e6);
    if (p.r1 == 0 || t < best * 0.995) { best = t; p.r1 = r; p.stages1 = st1; p.g1 = (int)ctas; }
  }
  if (p.r1 == 0) return fail(PMX_ERR_UNSUPPORTED, "dense_mlp: the stage does not fit in shared memory");
  p.f1 = (int)ceil_div(I, p.r1);
  const size_t stage2 = tok + 256 * 128;
  p.stages2 = (int)(budget / stage2);
  if (p.stages2 > 8) p.stages2 = 8;
  if (p.stages2 < 2) return fail(PMX_ERR_UNSUPPORTED, "dense_mlp: the stage does not fit in shared memory");
  p.g2 = full_round_grid(E * p.f2, sms);
  const size_t ring1 = (size_t)p.stages1 * (tok + 2 * (size_t)p.r1 * 128) + (size_t)(128 - p.r1) * 128;
  const size_t ring2 = (size_t)p.stages2 * stage2;
  p.ring_bytes = (int)(ring1 > ring2 ? ring1 : ring2);

  CUtensorMap mx, mwu, mh, mw2;
  int st = make_map(&mx, x, (uint64_t)T, (uint64_t)H, (uint32_t)p.tile_tok, dtype);
  if (st != PMX_OK) return st;
  st = make_map(&mwu, wu, (uint64_t)E * N, (uint64_t)H, (uint32_t)p.r1, dtype);
  if (st != PMX_OK) return st;
  st = make_map(&mh, h, (uint64_t)T * k, (uint64_t)I, (uint32_t)p.tile_tok, dtype);
  if (st != PMX_OK) return st;
  st = make_map(&mw2, w2, (uint64_t)E * H, (uint64_t)I, 128u, dtype);
  if (st != PMX_OK) return st;

  const size_t smem = fixed + (size_t)p.ring_bytes;
  const void* kern = dtype == PMX_DTYPE_BF16 ? (const void*)expert_mlp_decode_kernel<__nv_bfloat16>
                                             : (const void*)expert_mlp_decode_kernel<__half>;
  PMX_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int grid = p.g1 > p.g2 ? p.g1 : p.g2;
  void* args[] = {(void*)&mx, (void*)&mwu, (void*)&mh, (void*)&mw2, (void*)&p};
  return launch_pdl(kern, dim3(grid), dim3(kThreads), smem, s, args);
}

}  // namespace pmx
