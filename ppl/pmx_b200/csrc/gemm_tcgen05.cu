// Grouped expert GEMM on the 5th-generation tensor cores (sm_100a):
//   y[r,:] = x[r,:] . w[e]^T (+ bias[e])    for rows r owned by expert e,
// optionally with SwiGLU applied to the fp32 accumulator before the store.
//
// One persistent CTA per SM, three roles:
//   warp 0   : TMA producer.  cp.async.bulk.tensor (128-byte swizzle) of the
//              token tile and the weight tile of every k-block into a ring of
//              shared-memory stages, completion on mbarriers.
//   warp 1   : owns tensor memory and issues tcgen05.mma (kind::f16, fp32
//              accumulation in TMEM); tcgen05.commit releases ring stages and
//              publishes finished accumulators.
//   warps 2-5: epilogue.  tcgen05.ld of the accumulator, bias / SwiGLU / cast,
//              predicated global stores.  Two accumulator buffers in TMEM let
//              the epilogue of one tile overlap the MMAs of the next.
//
// Work items are (expert, token tile, feature tile, K slice).  The list is
// derived on the device from expert_offset, so there is no host
// synchronisation and the launch does not depend on the routing.  Items are
// ordered expert-major with the token tile fastest, so the CTAs running at
// one time share weight tiles through L2 and each weight byte leaves HBM once.
// The CTAs that take items are the smallest set that needs no more rounds of
// items than the cap allows (WorkIter::init), so every round is full; with
// stream_k the k-blocks of all items are dealt out evenly instead and tiles cut
// at a CTA boundary are completed through partial tiles in the workspace.
//
// Two operand assignments (template MODE):
//   0  tokens on MMA-M (128 rows), weight rows on MMA-N (up to 256): prefill.
//   1  weight rows on MMA-M (128), tokens on MMA-N (16..256): decode, where an
//      expert owns few rows and the weights are streamed once from HBM.
//
// Every wait on an mbarrier is bounded; a wait that runs out records where in
// the status words of the workspace, raises a CTA-wide abort flag and all
// roles drain and leave through the common exit (which frees the TMEM).
#include <cuda.h>
#include <cudaTypedefs.h>

#include <type_traits>

#include "common.cuh"

namespace pmx {
namespace {

#include "tcgen05_common.cuh"

template <typename T, int MODE, bool SWIGLU, bool DENSE = false, bool TWO = false>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x,
                       const __grid_constant__ CUtensorMap map_w,
                       const __grid_constant__ SmallBoxMaps map_ws, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tt = p.tile_tok, ft = p.tile_feat;
  const int wrows = SWIGLU ? 2 * ft : ft;            // weight rows per stage
  // weight rows on MMA-M without SwiGLU and ft = 256: two 128-row tiles of consecutive
  // features per stage (one 256-row copy, two MMAs, accumulator columns [0,tt) and [tt,2tt))
  // (a template flag: as a run-time test inside the MMA issuer's loop it made every launch of
  // the one-tile kernel slower, 69 against 49 us for the one-token down projection)
  constexpr bool two_tiles = TWO;
  static_assert(!TWO || (MODE == 1 && !SWIGLU && !DENSE), "two tiles per stage: weight rows on MMA-M, no SwiGLU");
  const uint32_t tok_bytes = tt * 128, w_bytes = wrows * 128;
  const uint32_t stage_bytes = tok_bytes + w_bytes;
  Shared* sh = reinterpret_cast<Shared*>(smem + (size_t)p.stages * stage_bytes);
  int* s_off = reinterpret_cast<int*>(sh + 1);       // [E+1] row offsets, clamped
  int* s_prefix = s_off + (p.E + 1);                 // [E+1] first work item of each expert
  int* s_rowmap = s_prefix + (p.E + 1);              // DENSE: [4 warps][128] output row of every token for the current expert

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- set-up ---------------------------------------------------------------
  // Everything up to pdl_wait() touches no memory another kernel writes, so under
  // programmatic dependent launch it overlaps the tail of the kernel in front.
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    stamp(p.stamps, 0);
    for (int i = 0; i < p.stages; ++i) {
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
    prefetch_tensormap(&map_w);
    if (MODE == 1 && p.balanced) {
#pragma unroll
      for (int i = 0; i < 4; ++i) prefetch_tensormap(&map_ws.m[i]);
    }
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  // Weights never depend on the kernel in front.  Guess that every expert owns rows that fit one
  // token tile (decode: true unless an expert is empty); the CTA's first item is then known from
  // the shapes alone, and the producer fills the ring with its weight tiles (no token tiles yet)
  // BEFORE the dependency wait.  A wrong guess costs nothing but those loads: the stages are
  // handed back unused.
  int pre_n = 0, pre_e = -1, pre_f0 = 0;
  const uint32_t smem_base = smem_u32(smem);
  if (MODE == 1 && !DENSE && p.prefetch && threadIdx.x == 0) {
    sh->discard = 0;
    WorkIter guess;
    guess.init(p, p.E);
    if (guess.next_item < guess.panel_end && guess.u_end - guess.u >= ft / 8) {
      pre_e = guess.next_item;
      pre_f0 = (int)guess.u * 8;
      pre_n = p.stages < p.kblocks ? p.stages : p.kblocks;
      const int wrow = pre_e * p.w_pitch + pre_f0;
      for (int st = 0; st < pre_n; ++st) {
        const uint32_t dst = smem_base + st * stage_bytes + tok_bytes;
        mbar_expect_tx_only(&sh->full[st], w_bytes);
        tma_load_2d(dst, &map_w, &sh->full[st], st * kBlockK, wrow);
        if (SWIGLU) tma_load_2d(dst + ft * 128, &map_w, &sh->full[st], st * kBlockK, wrow + p.N / 2);
      }
    }
  }
  if (DENSE) {
    // Every expert is applied to all p.M tokens (operand x itself, not the gathered rows), so
    // the work list does not depend on the routing and the loads and MMAs start while the
    // routing kernel in front of this one is still running; only the epilogue warps wait for
    // it (they need to know which token rows an expert owns, and where they go).
    for (int e = threadIdx.x; e <= p.E; e += blockDim.x) s_off[e] = e * p.M;
  } else {
    pdl_wait();
    // CTA 0 clears the status words (a failed wait is recorded no earlier than
    // its 2 s limit, long after this store)
    if (blockIdx.x == 0 && threadIdx.x < 4) p.status[threadIdx.x] = 0;
    for (int e = threadIdx.x; e <= p.E; e += blockDim.x) {
      long long o = offset_at(p.off, e, p.M);
      s_off[e] = (int)(o < 0 ? 0 : (o > p.M ? p.M : o));
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < p.E; ++e) {
      if (s_off[e + 1] < s_off[e]) s_off[e + 1] = s_off[e];  // keep it monotone
      s_prefix[e] = acc;
      const int rows = s_off[e + 1] - s_off[e];
      acc += ((rows + tt - 1) / tt) * p.feat_tiles * p.split_k;
    }
    s_prefix[p.E] = acc;
    if (MODE == 1 && !DENSE && p.prefetch && pre_n > 0) {
      // was the guess right?  compare it with the real first item of this CTA
      WorkIter real;
      Item first;
      int idx = 0;
      real.init(p, acc);
      const bool have = real.next(p, acc, s_off, s_prefix, first, idx);
      const bool hit = have && first.e == pre_e && first.f0 == pre_f0 && first.fn == ft && first.kb0 == 0 &&
                       first.kb1 >= pre_n;
      if (!hit) {
        sh->discard = pre_n;
        for (int st = 0; st < pre_n; ++st) mbar_arrive(&sh->full[st]);   // completes once the weights have landed
        pre_n = -pre_n;                                                  // negative: discarded
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  const int total_items = s_prefix[p.E];
  if (threadIdx.x == 0) stamp(p.stamps, 1);

  if (warp == 0) {
    // ========================= TMA producer =================================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int pre_left = pre_n > 0 ? pre_n : 0;     // stages that already hold the first item's weight tiles
      if (pre_n < 0) {                          // discarded stages: the ring starts behind them
        stage = -pre_n;
        if (stage == p.stages) { stage = 0; phase ^= 1u; }
      }
      Item it;
      int item = 0;
      WorkIter work;
      work.init(p, total_items);
      bool ok = true;
      // L2 prefetch: a second walk over this CTA's k-blocks, p.l2_ahead rounds in front of the
      // ring's own weight loads (whose first `stages` rounds are requested at once anyway)
      WorkIter ahead;
      Item ait;
      int aitem = 0, akb = 0;
      bool ahave = false;
      auto prefetch_step = [&](bool issue) {
        if (!ahave) return;
        if (issue) {
          const int arow = ait.e * p.w_pitch + ait.f0;
          tma_prefetch_l2_2d(&map_w, akb * kBlockK, arow);
          if (SWIGLU) tma_prefetch_l2_2d(&map_w, akb * kBlockK, arow + p.N / 2);
        }
        if (++akb >= ait.kb1) {
          ahave = ahead.next(p, total_items, s_off, s_prefix, ait, aitem);
          akb = ahave ? ait.kb0 : 0;
        }
      };
      if (MODE == 1 && p.l2_ahead > 0) {
        ahead.init(p, total_items);
        ahave = ahead.next(p, total_items, s_off, s_prefix, ait, aitem);
        akb = ahave ? ait.kb0 : 0;
        for (int i = 0; i < p.stages + p.l2_ahead; ++i) prefetch_step(i >= p.stages);
      }
      while (ok && work.next(p, total_items, s_off, s_prefix, it, item)) {
        if (DENSE) it.row0 = 0;
        const int wrow = it.e * p.w_pitch + it.f0;
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          if (MODE == 1 && p.l2_ahead > 0) prefetch_step(true);
          if (pre_left > 0) {
            // the weights of this k-block are in flight (or there) already: add the token tile
            --pre_left;
            mbar_expect_tx(&sh->full[stage], tok_bytes);
            tma_load_2d(smem_base + stage * stage_bytes, &map_x, &sh->full[stage], kb * kBlockK, it.row0);
            if (++stage == p.stages) { stage = 0; phase ^= 1u; }
            continue;
          }
          ok = wait_barrier(&sh->empty[stage], phase ^ 1u, sh, p.status, 0, item);
          if (!ok) break;
          const uint32_t dst = smem_base + stage * stage_bytes;
          if (MODE == 1 && p.balanced && it.fn != ft) {
            // a range of it.fn < 128 feature rows: boxes of 64, 32, 16 and 8 rows (each at
            // most once); the rows of the stage behind them keep stale data that only
            // reaches accumulator lanes nobody stores
            mbar_expect_tx(&sh->full[stage], tok_bytes + (SWIGLU ? 2u : 1u) * (uint32_t)it.fn * 128u);
            tma_load_2d(dst, &map_x, &sh->full[stage], kb * kBlockK, it.row0);
            int done = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const int rows = 64 >> b;
              if (it.fn - done >= rows) {
                tma_load_2d(dst + tok_bytes + done * 128, &map_ws.m[b], &sh->full[stage], kb * kBlockK, wrow + done);
                if (SWIGLU)
                  tma_load_2d(dst + tok_bytes + (ft + done) * 128, &map_ws.m[b], &sh->full[stage], kb * kBlockK,
                              wrow + p.N / 2 + done);
                done += rows;
              }
            }
          } else {
            mbar_expect_tx(&sh->full[stage], stage_bytes);
            tma_load_2d(dst, &map_x, &sh->full[stage], kb * kBlockK, it.row0);
            tma_load_2d(dst + tok_bytes, &map_w, &sh->full[stage], kb * kBlockK, wrow);
            if (SWIGLU)
              tma_load_2d(dst + tok_bytes + ft * 128, &map_w, &sh->full[stage], kb * kBlockK,
                          wrow + p.N / 2);
          }
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
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
      const uint32_t idesc = make_idesc<T>(128, MODE == 0 ? wrows : tt);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      Item it;
      int item = 0;
      WorkIter work;
      work.init(p, total_items);
      bool ok = true;
      bool first_tile = true;
      if (MODE == 1 && !DENSE && p.prefetch) {
        // stages the producer filled for an item this CTA does not have: wait for the copies, hand them back
        for (int d = sh->discard; d > 0 && ok; --d) {
          ok = wait_barrier(&sh->full[stage], phase, sh, p.status, 2, -1);
          if (!ok) break;
          mbar_arrive(&sh->empty[stage]);
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
      }
      while (ok && work.next(p, total_items, s_off, s_prefix, it, item)) {
        ok = wait_barrier(&sh->acc_empty[acc], acc_phase ^ 1u, sh, p.status, 1, item);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kAccStride;
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          ok = wait_barrier(&sh->full[stage], phase, sh, p.status, 2, item);
          if (!ok) break;
          if (p.stamps && first_tile) { stamp(p.stamps, 2); first_tile = false; }
          tc_fence_after();
          const uint32_t tok_addr = smem_base + stage * stage_bytes;
          const uint32_t w_addr = tok_addr + tok_bytes;
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
            const uint32_t koff = kk * kUmmaK * 2;  // bytes inside the 128-byte row
            const uint32_t accum = (kb > it.kb0 || kk > 0) ? 1u : 0u;
            if (MODE == 0) {
              umma_f16(d_tmem, smem_desc_sw128(tok_addr + koff), smem_desc_sw128(w_addr + koff), idesc, accum);
            } else {
              const uint64_t bdesc = smem_desc_sw128(tok_addr + koff);
              umma_f16(d_tmem, smem_desc_sw128(w_addr + koff), bdesc, idesc, accum);
              if (SWIGLU || two_tiles)
                umma_f16(d_tmem + tt, smem_desc_sw128(w_addr + 128 * 128 + koff), bdesc, idesc, accum);
            }
          }
          umma_commit(&sh->empty[stage]);  // stage reusable once these MMAs have read it
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&sh->acc_full[acc]);   // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
      stamp(p.stamps, 3);
    }
  } else {
    // ========================= epilogue (warps 2..5) ========================
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    Item it;
    int item = 0;
    WorkIter work;
    work.init(p, total_items);
    bool ok = true;
    const bool partial = p.split_k > 1;
    T* y = reinterpret_cast<T*>(p.y);
    float* yp = reinterpret_cast<float*>(p.y);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    const int acc_cols = MODE == 0 ? wrows : (SWIGLU || two_tiles ? 2 * tt : tt);   // accumulator columns in use
    int map_expert = -1;
    if (DENSE) {
      pdl_wait();   // the routing (invert_permutation, expert_offset) is complete from here on
      if (blockIdx.x == 0 && warp == 2 && lane < 4) p.status[lane] = 0;
    }
    if (warp == 2 && lane == 0) stamp(p.stamps, 4);
    while (work.next(p, total_items, s_off, s_prefix, it, item)) {
      if (DENSE) {
        it.row0 = 0;
        it.row_end = p.M;
        if (it.e != map_expert) {
          // which row of the expert-sorted output holds token t for this expert (-1: not routed
          // here); every epilogue warp keeps its own copy, so no warp waits for another
          __syncwarp();
          const long long lo = p.off[it.e], hi = p.off[it.e + 1];
          for (int t = lane; t < 128; t += 32) {
            int r = -1;
            if (t < p.M) {
              for (int j = 0; j < p.k; ++j) {
                const long long v = p.inv[(long long)t * p.k + j];
                if (v >= lo && v < hi) r = (int)v;
              }
            }
            s_rowmap[q * 128 + t] = r;
          }
          __syncwarp();
          map_expert = it.e;
        }
      }
      ok = wait_barrier(&sh->acc_full[acc], acc_phase, sh, p.status, 3, item);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      if (warp == 2 && lane == 0) stamp(p.stamps, 7);   // (last item: its accumulator is complete)
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * kAccStride + (static_cast<uint32_t>(q * 32) << 16);
      if (p.stream_k && it.kb0 > 0) {
        // partial tile: raw accumulators -> this CTA's slot, then one count per warp
        float* slot = p.sk_slots + (size_t)blockIdx.x * (256 * 128) + q * 32 + lane;
        for (int c = 0; c < acc_cols; c += 16) {
          float g[16];
          __syncwarp();
          tmem_ld16(taddr + c, g);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) slot[(size_t)(c + i) * 128] = g[i];
        }
        __threadfence();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          atomicAdd(p.sk_flags + blockIdx.x, 1);
          mbar_arrive(&sh->acc_empty[acc]);
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        continue;
      }
      if (p.stream_k && it.kb1 < p.kblocks) {
        // owner of a tile whose remaining k-blocks went to the following CTAs:
        // add their partial tiles to the accumulator in tensor memory
        const long long item_end = ((long long)item + 1) * p.kblocks;
        for (int c2 = blockIdx.x + 1; c2 < work.grid && (long long)c2 * work.units / work.grid < item_end; ++c2) {
          // a CTA whose share of the units is empty has nothing to contribute
          if ((long long)(c2 + 1) * work.units / work.grid == (long long)c2 * work.units / work.grid) continue;
          if (lane == 0) {
            const unsigned long long t_start = global_ns();
            unsigned int spins = 0;
            while (ld_acquire_gpu_s32(p.sk_flags + c2) < 4) {
              if ((++spins & 255u) == 0u) {
                if (sh->abort) break;
                if (global_ns() - t_start > kWaitLimitNs) {
                  sh->abort = 1;
                  if (atomicExch(p.status, 1) != 1) { p.status[1] = 4; p.status[2] = item; p.status[3] = c2; }
                  break;
                }
              }
            }
          }
          __syncwarp();
          const float* slot = p.sk_slots + (size_t)c2 * (256 * 128) + q * 32 + lane;
          for (int c = 0; c < acc_cols; c += 16) {
            float g[16];
            __syncwarp();
            tmem_ld16(taddr + c, g);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) g[i] += __ldcg(slot + (size_t)(c + i) * 128);
            tmem_st16(taddr + c, g);
          }
          tmem_wait_st();
        }
        __syncwarp();
      }
      if (MODE == 0) {
        const int row = it.row0 + q * 32 + lane;
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
          if (partial) {
            float* dst = yp + ((int64_t)it.ks * p.M + row) * p.n_out + col;
            if (col + 16 <= p.n_out) {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                reinterpret_cast<float4*>(dst)[i] = make_float4(g[4 * i], g[4 * i + 1], g[4 * i + 2], g[4 * i + 3]);
            } else {
              for (int i = 0; i < 16 && col + i < p.n_out; ++i) dst[i] = g[i];
            }
          } else {
            T* dst = y + (int64_t)row * p.n_out + col;
            if (col + 16 <= p.n_out) {
              store16<T>(dst, g);
            } else {
              for (int i = 0; i < 16 && col + i < p.n_out; ++i) dst[i] = Elem<T>::from_f(g[i]);
            }
          }
        };
        // 32 columns per round: the tensor-memory loads of both halves are in flight before
        // the one wait, so a short-K tile's epilogue is not a chain of load latencies
        for (int c = 0; c < ft; c += 32) {
          const bool two = c + 32 <= ft;
          float g0[16], g1[16], u0[16], u1[16];
          __syncwarp();  // tcgen05.ld is warp-collective: keep the lanes together
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
      } else {
        const int f = it.f0 + q * 32 + lane;  // output feature of this thread
        const bool f_ok = f < p.n_out && q * 32 + lane < it.fn;
        const int f2 = f + 128;               // two tiles per stage: its feature in the second tile
        const bool f2_ok = two_tiles && f2 < p.n_out && q * 32 + lane + 128 < it.fn;
        float bg = 0.f, bu = 0.f;
        if (bias && f_ok) {
          bg = Elem<T>::to_f(bias[(int64_t)it.e * p.w_pitch + f]);
          if (SWIGLU) bu = Elem<T>::to_f(bias[(int64_t)it.e * p.w_pitch + p.n_out + f]);
        }
        if (bias && f2_ok) bu = Elem<T>::to_f(bias[(int64_t)it.e * p.w_pitch + f2]);
        // up to 32 token columns per round: their tensor-memory loads are all in flight before
        // the one wait (a tcgen05.ld round trip costs several hundred ns).  Not more: the
        // registers of 64 columns would keep a CTA of this kernel from sharing an SM with a
        // CTA of the routing kernel (two warps of each per sub-partition's register file).
        for (int c = 0; c < tt; c += 32) {
          if (it.row0 + c >= it.row_end || q * 32 >= it.fn) break;  // same for the whole warp
          float g[2][16], u[2][16];
          __syncwarp();
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            if (c + ch * 16 < tt && it.row0 + c + ch * 16 < it.row_end) {
              tmem_ld16(taddr + c + ch * 16, g[ch]);
              if (SWIGLU || two_tiles) tmem_ld16(taddr + tt + c + ch * 16, u[ch]);
            }
          }
          tmem_wait_ld();
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            if (c + ch * 16 < tt && it.row0 + c + ch * 16 < it.row_end) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const int row = DENSE ? s_rowmap[q * 128 + c + ch * 16 + i] : it.row0 + c + ch * 16 + i;
                if ((DENSE ? row >= 0 : row < it.row_end) && f_ok) {
                  float v = g[ch][i] + bg;
                  if (SWIGLU) v = swiglu_f(v, u[ch][i] + bu, p.beta);
                  if (partial)
                    yp[((int64_t)it.ks * p.M + row) * p.n_out + f] = v;
                  else
                    y[(int64_t)row * p.n_out + f] = Elem<T>::from_f(v);
                }
                if (!DENSE && row < it.row_end && f2_ok) {
                  const float v = u[ch][i] + bu;
                  if (partial)
                    yp[((int64_t)it.ks * p.M + row) * p.n_out + f2] = v;
                  else
                    y[(int64_t)row * p.n_out + f2] = Elem<T>::from_f(v);
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->acc_empty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
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
}

// ----------------------------------------------------------------------------- host side
constexpr size_t kRowMapBytes = 4 * 128 * sizeof(int);   // the dense variant's token -> row maps

size_t smem_bytes_for(const TcPlan& plan, bool swiglu, int E) {
  const size_t stage = (size_t)(plan.tile_tok + (swiglu ? 2 : 1) * plan.tile_feat) * 128;
  return 1024 + stage * plan.stages + sizeof(Shared) + 2 * (size_t)(E + 1) * sizeof(int) + kRowMapBytes;
}

template <typename T, int MODE, bool SWIGLU, bool TWO = false>
int launch_inst(const CUtensorMap& mx, const CUtensorMap& mw, const SmallBoxMaps& mws, const Params& p, int grid,
                size_t smem, cudaStream_t s) {
  auto kern = grouped_gemm_tc_kernel<T, MODE, SWIGLU, false, TWO>;
  PMX_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  void* args[] = {(void*)&mx, (void*)&mw, (void*)&mws, (void*)&p};
  return launch_pdl((const void*)kern, dim3(grid), dim3(kThreads), smem, s, args);
}

int pow2_at_least(int64_t v, int lo, int hi) {
  int r = lo;
  while (r < v && r < hi) r <<= 1;
  return r;
}

}  // namespace

bool plan_gemm_tc(int64_t M, int64_t N, int64_t K, int E, int dtype, int epilogue,
                  const pmx_gemm_plan* user, TcPlan* plan) {
  const bool swiglu = epilogue == PMX_EPILOGUE_SWIGLU;
  const int64_t n_out = swiglu ? N / 2 : N;
  if (dtype != PMX_DTYPE_F16 && dtype != PMX_DTYPE_BF16) return false;
  if (K % 8 || n_out % 8 || K < 8 || E > kMaxExperts) return false;
  if (M >= (1ll << 31) || (int64_t)E * N >= (1ll << 31) || M * n_out >= (1ll << 40)) return false;
  const int sms = sm_count();
  TcPlan pl{};
  const double avg_rows = (double)M / E;
  pl.kernel = user && user->kernel ? user->kernel : (avg_rows >= 96.0 ? PMX_GEMM_TC_TOKENS_M : PMX_GEMM_TC_WEIGHTS_M);
  if (pl.kernel != PMX_GEMM_TC_TOKENS_M && pl.kernel != PMX_GEMM_TC_WEIGHTS_M) return false;
  if (pl.kernel == PMX_GEMM_TC_TOKENS_M) {
    pl.tile_tok = 128;
    const int ft_max = swiglu ? 128 : 256;
    pl.tile_feat = user && user->tile_feat ? user->tile_feat : pow2_at_least(n_out, 16, ft_max);
    if (pl.tile_feat % 16 || pl.tile_feat < 16 || pl.tile_feat > ft_max) return false;
  } else {
    pl.tile_feat = 128;
    const int tt_max = swiglu ? 128 : 256;
    const int64_t est = (int64_t)(avg_rows * 1.5) + 1;
    pl.tile_tok = user && user->tile_tok ? user->tile_tok : pow2_at_least(est < M ? est : M, 16, tt_max);
    if (pl.tile_tok % 16 || pl.tile_tok < 16 || pl.tile_tok > tt_max) return false;
  }
  const int kblocks = (int)ceil_div(K, kBlockK);
  const int64_t feat_tiles = ceil_div(n_out, pl.tile_feat);
  const int want_sk = user ? user->stream_k : 0;
  // Weight rows on MMA-M: deal the feature rows of all panels out evenly (8-row units)
  // instead of whole 128-row tiles, unless the caller asks for whole tiles or stream-K.
  pl.l2_ahead = user && user->l2_prefetch ? (user->l2_prefetch < 0 ? 0 : user->l2_prefetch) : default_l2_prefetch();
  pl.balanced = pl.kernel == PMX_GEMM_TC_WEIGHTS_M && want_sk != 1 && !(user && user->balance == 2) ? 1 : 0;
  if (user && user->split_k) {
    pl.split_k = user->split_k;
  } else if (want_sk == 1) {
    pl.split_k = 1;   // stream-K slices K itself
  } else {
    pl.split_k = 1;
    // experts with at least one row (estimate) x token tiles each
    const int64_t act = M < E ? M : E;
    const int64_t tok_tiles = act * (int64_t)ceil_div((int64_t)(avg_rows < 1 ? 1 : avg_rows), pl.tile_tok);
    const int64_t items = tok_tiles * feat_tiles;
    // Whole tiles: K is sliced when there are fewer tiles than half the SMs (one token, or a
    // thin tensor-parallel shard).  Evenly dealt rows: a CTA's time is set by its k-block
    // rounds, and rounds that carry few rows put few bytes in flight, so K is sliced when a
    // CTA would get at most half a 128-row tile, until it gets about a whole one.  With
    // SwiGLU the kernel then produces plain [gate | up] partial sums and the activation
    // moves into the final sum.
    const int64_t ctas = sms < 128 ? sms : 128;
    const bool slice = pl.balanced ? 2 * tok_tiles * (n_out / 8) <= 16 * ctas : 2 * items <= sms;
    if (slice) {
      int64_t want;
      if (pl.balanced) {
        const int64_t units = tok_tiles * (N / 8);
        want = 16 * ctas / (units > 0 ? units : 1);
      } else {
        const int64_t base = swiglu ? tok_tiles * ceil_div(N, pl.tile_feat) : items;
        want = ceil_div(2 * sms, base);
      }
      const int64_t cap = kblocks / 8 > 0 ? kblocks / 8 : 1;
      if (want > cap) want = cap;
      if (want > 16) want = 16;
      if (want < 1) want = 1;
      pl.split_k = (int)want;
    }
  }
  if (pl.split_k < 1) return false;
  if (pl.split_k > kblocks) pl.split_k = kblocks;
  {
    const int per = (int)ceil_div(kblocks, pl.split_k);
    pl.split_k = (int)ceil_div(kblocks, per);  // no empty slice
  }
  if (pl.split_k > 1 && n_out % 4) return false;
  const bool kernel_swiglu = swiglu && pl.split_k == 1;
  // Weight rows on MMA-M without the SwiGLU epilogue (down projection, dense linears): a stage
  // of 128 rows is 16 KB, and a CTA's time is set by its number of k-block rounds (producer
  // and MMA threads are single threads), so when every working CTA has at least 256 rows of
  // one panel the stage holds two 128-row tiles: half as many rounds for the same bytes.
  if (pl.kernel == PMX_GEMM_TC_WEIGHTS_M && !swiglu && pl.split_k == 1 && pl.balanced && want_sk != 1 &&
      !(user && user->tile_feat) && pl.tile_tok <= 128 && n_out % 256 == 0) {
    const int64_t act = M < E ? M : E;
    const int64_t panels = act * (int64_t)ceil_div((int64_t)(avg_rows < 1 ? 1 : avg_rows), pl.tile_tok);
    const int64_t ctas = sms < 128 ? sms : 128;
    if (panels * (n_out / 8) >= 32 * ctas) pl.tile_feat = 256;
  }
  if (!kernel_swiglu && pl.kernel == PMX_GEMM_TC_TOKENS_M && !(user && user->tile_feat) && swiglu)
    pl.tile_feat = pow2_at_least(N, 16, 256);
  const size_t stage = (size_t)(pl.tile_tok + (kernel_swiglu ? 2 : 1) * pl.tile_feat) * 128;
  const size_t fixed = 1024 + sizeof(Shared) + 2 * (size_t)(E + 1) * sizeof(int) + kRowMapBytes;
  int st = (int)((227 * 1024 - fixed) / stage);
  if (st > kMaxStages) st = kMaxStages;
  if (user && user->stages) st = user->stages < st ? user->stages : st;
  if (st < 2) return false;
  pl.stages = st;
  pl.max_ctas = user && user->max_ctas ? user->max_ctas : sms;
  // Weight streaming is HBM-bound: 128 CTAs with full rings in flight saturate the memory
  // system, and more CTAs only add rounds that are no shorter (measured on B200: 6.5-6.7
  // TB/s with 128 CTAs against 6.3 with all 148 SMs); the tensor-bound assignment uses every SM.
  pl.cta_cap = pl.max_ctas;
  if (!(user && user->max_ctas) && pl.kernel == PMX_GEMM_TC_WEIGHTS_M && pl.cta_cap > 128) pl.cta_cap = 128;
  if (user && user->cta_cap > 0 && user->cta_cap <= pl.max_ctas) pl.cta_cap = user->cta_cap;
  pl.full_rounds = !(user && user->full_rounds == 2);
  // Stream-K (k-blocks of all items dealt out evenly over the CTAs) is available on
  // request.  Measured on B200 it does not beat whole tiles on a grid sized to
  // full rounds (see WorkIter::init): 283 vs 290 us for the Mixtral gate/up
  // projection at 64 tokens, but 55 vs 46 us on a 1/8 tensor-parallel shard.
  pl.stream_k = pl.split_k == 1 && want_sk == 1 ? 1 : 0;
  if (want_sk == 1 && !pl.stream_k) return false;
  // Stream-K: the owner of a cut tile waits for CTAs with higher indices, so all CTAs of
  // the launch have to be resident together: one per SM and the SMs not shared with other
  // kernels.  A ring so small that two CTAs fit on one SM is refused (the second would
  // block in the tensor-memory allocation until the first exits).
  if (pl.stream_k && fixed + stage * (size_t)pl.stages <= 114 * 1024) return false;
  *plan = pl;
  return true;
}

size_t gemm_tc_workspace_bytes(int64_t M, int64_t N, int epilogue, const TcPlan& plan) {
  size_t b = kStatusBytes;
  // split-K partial sums cover all N accumulator columns (SwiGLU is then applied in the final sum)
  if (plan.split_k > 1) b += (size_t)plan.split_k * M * N * sizeof(float);
  // stream-K: one flag and one 256-column x 128-lane fp32 partial tile per CTA
  if (plan.stream_k) b += kStreamKFlagBytes + (size_t)plan.max_ctas * 256 * 128 * sizeof(float);
  (void)epilogue;
  return b;
}

int launch_gemm_tc(const void* x, const int64_t* off, const void* w, const void* bias, void* y,
                   int64_t M, int64_t N, int64_t K, int E, int dtype, int epilogue, float beta,
                   const TcPlan& plan, void* ws, size_t ws_bytes, cudaStream_t s) {
  const bool swiglu_any = epilogue == PMX_EPILOGUE_SWIGLU;
  const bool swiglu = swiglu_any && plan.split_k == 1;   // SwiGLU inside the kernel's epilogue
  const int64_t n_out = swiglu ? N / 2 : N;               // accumulator columns the kernel stores
  if (!aligned16(x) || !aligned16(w) || !aligned16(y))
    return fail(PMX_ERR_ALIGNMENT, "grouped_linear: x, w and y must be 16-byte aligned");
  const size_t need = gemm_tc_workspace_bytes(M, N, epilogue, plan);
  if (!ws || ws_bytes < need) return fail(PMX_ERR_WORKSPACE, "grouped_linear: workspace of %zu bytes needed, %zu given", need, ws_bytes);
  if (!aligned16(ws)) return fail(PMX_ERR_ALIGNMENT, "grouped_linear: workspace must be 16-byte aligned");

  CUtensorMap mx, mw;
  int st = make_map(&mx, x, (uint64_t)M, (uint64_t)K, (uint32_t)plan.tile_tok, dtype);
  if (st != PMX_OK) return st;
  st = make_map(&mw, w, (uint64_t)(E - 1) * (uint64_t)(plan.w_pitch > 0 ? plan.w_pitch : N) + (uint64_t)N, (uint64_t)K, (uint32_t)plan.tile_feat, dtype);
  if (st != PMX_OK) return st;

  SmallBoxMaps mws{};
  if (plan.balanced) {
    for (int b = 0; b < 4; ++b) {
      st = make_map(&mws.m[b], w, (uint64_t)(E - 1) * (uint64_t)(plan.w_pitch > 0 ? plan.w_pitch : N) + (uint64_t)N, (uint64_t)K, (uint32_t)(64 >> b), dtype);
      if (st != PMX_OK) return st;
    }
  }
  Params p{};
  p.off = off;
  p.bias = plan.split_k > 1 ? nullptr : bias;  // with split-K the bias joins in the final sum
  p.status = reinterpret_cast<int*>(ws);
  p.y = plan.split_k > 1 ? reinterpret_cast<void*>(reinterpret_cast<char*>(ws) + kStatusBytes) : y;
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.E = E;
  p.w_pitch = plan.w_pitch > 0 ? plan.w_pitch : (int)N;
  p.n_out = (int)n_out;
  p.tile_tok = plan.tile_tok;
  p.tile_feat = plan.tile_feat;
  p.feat_tiles = plan.balanced ? 1 : (int)ceil_div(n_out, plan.tile_feat);
  p.balanced = plan.balanced;
  p.prefetch = weight_prefetch_enabled() && plan.kernel == PMX_GEMM_TC_WEIGHTS_M && plan.balanced && plan.split_k == 1 && !plan.stream_k &&
               n_out >= 128;
  p.units_per_panel = (int)(n_out / 8);
  p.l2_ahead = plan.kernel == PMX_GEMM_TC_WEIGHTS_M && !plan.stream_k ? plan.l2_ahead : 0;
  p.stamps = next_stamp_slot(2);
  p.kblocks = (int)ceil_div(K, kBlockK);
  p.split_k = plan.split_k;
  p.kb_per_split = (int)ceil_div(p.kblocks, plan.split_k);
  p.stages = plan.stages;
  p.beta = beta;
  p.stream_k = plan.stream_k;
  p.cta_cap = plan.cta_cap;
  p.full_rounds = plan.full_rounds;
  if (plan.stream_k) {
    if (plan.max_ctas > 256) return fail(PMX_ERR_UNSUPPORTED, "grouped_linear: stream-K supports at most 256 CTAs");
    char* base = reinterpret_cast<char*>(ws) + kStatusBytes;
    p.sk_flags = reinterpret_cast<int*>(base);
    p.sk_slots = reinterpret_cast<float*>(base + kStreamKFlagBytes);
    PMX_CUDA_OK(cudaMemsetAsync(p.sk_flags, 0, kStreamKFlagBytes, s));
  }

  const size_t smem = smem_bytes_for(plan, swiglu, E);
  const int grid = plan.max_ctas;
  const bool bf = dtype == PMX_DTYPE_BF16;
  const int mode = plan.kernel == PMX_GEMM_TC_TOKENS_M ? 0 : 1;
#define PMX_TC_LAUNCH(TT, MD, SW) st = launch_inst<TT, MD, SW>(mx, mw, mws, p, grid, smem, s)
  if (mode == 0) {
    if (swiglu) { if (bf) PMX_TC_LAUNCH(__nv_bfloat16, 0, true); else PMX_TC_LAUNCH(__half, 0, true); }
    else        { if (bf) PMX_TC_LAUNCH(__nv_bfloat16, 0, false); else PMX_TC_LAUNCH(__half, 0, false); }
  } else {
    if (swiglu) { if (bf) PMX_TC_LAUNCH(__nv_bfloat16, 1, true); else PMX_TC_LAUNCH(__half, 1, true); }
    else if (plan.tile_feat == 256) {
      if (bf) st = launch_inst<__nv_bfloat16, 1, false, true>(mx, mw, mws, p, grid, smem, s);
      else st = launch_inst<__half, 1, false, true>(mx, mw, mws, p, grid, smem, s);
    }
    else        { if (bf) PMX_TC_LAUNCH(__nv_bfloat16, 1, false); else PMX_TC_LAUNCH(__half, 1, false); }
  }
#undef PMX_TC_LAUNCH
  if (st != PMX_OK) return st;
  if (plan.split_k > 1)
    return launch_splitk_finish(reinterpret_cast<const float*>(p.y), off, bias, y, M,
                                swiglu_any ? N / 2 : N, E, plan.split_k, dtype, swiglu_any, beta, s);
  return PMX_OK;
}

// ----------------------------------------------------------------------------- dense gate/up
// h[row(t,e), :] = SwiGLU(x[t] . w[e]^T (+ bias[e])) for every token t routed to expert e, with
// the products computed for ALL tokens against every expert (weights on MMA-M, the T tokens on
// MMA-N): the kernel's loads and MMAs need nothing from the routing, so under programmatic
// dependent launch they overlap the routing kernel in front; only the epilogue waits for it.
bool dense_gate_up_covers(int64_t T, int64_t N, int64_t K, int E, int k, int dtype) {
  return T >= 1 && T <= 128 && E >= 1 && E <= kMaxExperts && k >= 1 && k <= E && K % 8 == 0 && K >= 8 && N % 16 == 0 &&
         (dtype == PMX_DTYPE_F16 || dtype == PMX_DTYPE_BF16) && (int64_t)E * N < (1ll << 31);
}

int launch_gemm_tc_dense(const void* x, const int64_t* inv, const int64_t* off, const void* w, const void* bias,
                         void* h, int64_t T, int64_t N, int64_t K, int E, int k, int dtype, float beta, void* ws,
                         size_t ws_bytes, cudaStream_t s) {
  if (!x || !inv || !off || !w || !h) return fail(PMX_ERR_INVALID_ARGUMENT, "dense_gate_up: null pointer");
  if (!dense_gate_up_covers(T, N, K, E, k, dtype))
    return fail(PMX_ERR_UNSUPPORTED, "dense_gate_up: covers 1..128 tokens, float16 / bfloat16, K a multiple of 8 and N of 16 (T=%lld N=%lld K=%lld)", (long long)T, (long long)N, (long long)K);
  if (!aligned16(x) || !aligned16(w) || !aligned16(h)) return fail(PMX_ERR_ALIGNMENT, "dense_gate_up: x, w and h must be 16-byte aligned");
  if (!ws || ws_bytes < kStatusBytes || !aligned16(ws))
    return fail(PMX_ERR_WORKSPACE, "dense_gate_up: a 16-byte aligned workspace of %zu bytes is needed", kStatusBytes);
  TcPlan plan{};
  plan.kernel = PMX_GEMM_TC_WEIGHTS_M;
  plan.tile_feat = 128;
  plan.tile_tok = (int)(ceil_div(T, 16) * 16);
  plan.split_k = 1;
  plan.balanced = 1;
  plan.full_rounds = 1;
  const int sms = sm_count();
  plan.max_ctas = sms;
  plan.cta_cap = sms < 128 ? sms : 128;
  const size_t stage = (size_t)(plan.tile_tok + 2 * plan.tile_feat) * 128;
  const size_t fixed = 1024 + sizeof(Shared) + 2 * (size_t)(E + 1) * sizeof(int) + kRowMapBytes;
  // 24 KB of every SM's shared memory stay free, so that a CTA of the routing kernel and a
  // CTA of this one fit on an SM together
  int st_n = (int)((203 * 1024 - fixed) / stage);
  if (st_n > kMaxStages) st_n = kMaxStages;
  if (st_n < 2) return fail(PMX_ERR_UNSUPPORTED, "dense_gate_up: the stage does not fit in shared memory");
  plan.stages = st_n;

  const int64_t n_out = N / 2;
  CUtensorMap mx, mw;
  int st = make_map(&mx, x, (uint64_t)T, (uint64_t)K, (uint32_t)plan.tile_tok, dtype);
  if (st != PMX_OK) return st;
  st = make_map(&mw, w, (uint64_t)E * N, (uint64_t)K, 128u, dtype);
  if (st != PMX_OK) return st;
  SmallBoxMaps mws{};
  for (int b = 0; b < 4; ++b) {
    st = make_map(&mws.m[b], w, (uint64_t)E * N, (uint64_t)K, (uint32_t)(64 >> b), dtype);
    if (st != PMX_OK) return st;
  }
  Params p{};
  p.off = off;
  p.inv = inv;
  p.k = k;
  p.bias = bias;
  p.status = reinterpret_cast<int*>(ws);
  p.y = h;
  p.M = (int)T; p.N = (int)N; p.K = (int)K; p.E = E;
  p.w_pitch = (int)N;
  p.n_out = (int)n_out;
  p.tile_tok = plan.tile_tok;
  p.tile_feat = 128;
  p.feat_tiles = 1;
  p.balanced = 1;
  p.units_per_panel = (int)(n_out / 8);
  p.l2_ahead = default_l2_prefetch();
  p.stamps = next_stamp_slot(3);
  p.kblocks = (int)ceil_div(K, kBlockK);
  p.split_k = 1;
  p.kb_per_split = p.kblocks;
  p.stages = plan.stages;
  p.beta = beta;
  p.cta_cap = plan.cta_cap;
  p.full_rounds = 1;
  const size_t smem = smem_bytes_for(plan, true, E);
  const void* kern = dtype == PMX_DTYPE_BF16 ? (const void*)grouped_gemm_tc_kernel<__nv_bfloat16, 1, true, true>
                                             : (const void*)grouped_gemm_tc_kernel<__half, 1, true, true>;
  PMX_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  void* args[] = {(void*)&mx, (void*)&mw, (void*)&mws, (void*)&p};
  return launch_pdl(kern, dim3(plan.max_ctas), dim3(kThreads), smem, s, args);
}

}  // namespace pmx
