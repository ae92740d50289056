// Decode-step attention over the key/value cache, one new token per sequence.
//
// Replaces, for decode steps, what dynamic_batching.MultiHeadCacheAttention.forward does
// with one Python loop body per sequence (torch_function/dynamic_batching/
// MultiHeadCacheAttention.py:104-130): KeyValueCache.forward stores the new key and value
// of every sequence into the cache and gathers the cached rows
// (dynamic_batching/KeyValueCache.py:86-138, cache_mode 0, no quantisation), and
// MultiHeadAttention.forward computes softmax(q . K^T / sqrt(d)) . V per sequence with
// grouped-query head sharing (dynamic_batching/MultiHeadAttention.py:54-108).
//
// HBM-bound: every cached key and value of the layer is read once.  The work is split over
// (sequence, kv head, slice of the cached positions); a CTA streams its slice once for all
// query heads that share the kv head with 16-byte loads (a warp fetches 2 or 4 head rows per
// instruction, several instructions in flight), with the running maximum / sum / weighted
// value sum of an online softmax in registers.  The slices of a (sequence, kv head) are merged by a second,
// tiny kernel.  All cache layouts of cache_mode 0 are covered through strides.
#include <atomic>
#include <type_traits>

#include "common.cuh"

namespace pmx {
namespace {

__device__ __forceinline__ uint32_t smem_u32_attn(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

constexpr int kAttnWarps = 4;
constexpr int kGroupLimit = 8;     // query heads per kv head
constexpr int kUnroll = 4;         // cached positions a warp works on per round

struct AttnParams {
  const void* q;        // [B, Hq, D]
  const void* k_cur;    // [B, Hkv, D]
  const void* v_cur;    // [B, Hkv, D]
  void* cache;          // element (row, kv, head, d) at layer_off + row*row_stride + kv*kv_stride + head*head_stride + d
  const int64_t* cachestarts;   // [B] first cache row of each sequence
  const int64_t* start_pos;     // [B] tokens already cached = position of the new token
  void* out;            // [B, Hq, D]
  float* part;          // [B, Hkv, splits, G, D + 2] partial sums (acc, max, sum)
  int64_t layer_off, row_stride, kv_stride, head_stride;
  int B, Hq, Hkv, splits, chunk;
  float scale;
};

// A head row (D 16-bit values) is read by D/8 lanes with one 16-byte load each, so a warp
// fetches 32/(D/8) positions per load instruction (2 for D = 128, 4 for D = 64).  Every such
// group of lanes runs its own online softmax over the positions it sees; the groups of a
// warp are merged with shuffles, the warps of the CTA through shared memory.
template <typename T, int D, int GMAX>   // GMAX: query heads per kv head the registers are sized for (>= the actual number)
__global__ void __launch_bounds__(kAttnWarps * 32, 3)
decode_attention_kernel(const AttnParams p) {
  constexpr int kMaxGroup = GMAX;
  constexpr int LPP = D / 8;          // lanes per position
  constexpr int PPL = 32 / LPP;       // positions per load instruction of a warp
  const int b = blockIdx.x, h = blockIdx.y, s = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / LPP, sl = lane % LPP;      // which position of the load, which 8 dims of the row
  const int G = p.Hq / p.Hkv;
  __shared__ float sm_acc[kAttnWarps][kMaxGroup][D];
  __shared__ float sm_m[kAttnWarps][kMaxGroup], sm_l[kAttnWarps][kMaxGroup];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t pos_new = p.start_pos[b];         // the new token's position; kv length = pos_new + 1
  const int64_t kvlen = pos_new + 1;
  const int64_t row0 = p.cachestarts[b];
  const T* q = reinterpret_cast<const T*>(p.q) + ((int64_t)b * p.Hq + (int64_t)h * G) * D;
  T* cache = reinterpret_cast<T*>(p.cache);
  const int64_t base = p.layer_off + (int64_t)h * p.head_stride + sl * 8;

  // this lane's 8 dims of every query of the group, pre-scaled
  float qv[kMaxGroup][8];
#pragma unroll
  for (int g = 0; g < kMaxGroup; ++g) {
    if (g < G) {
      float f[8];
      unpack16<T>(ld_stream16(q + (int64_t)g * D + sl * 8), f);
#pragma unroll
      for (int v = 0; v < 8; ++v) qv[g][v] = f[v] * p.scale;
    }
  }
  // the new key / value of this sequence and kv head: stored into the cache by the CTA of
  // slice 0 and taken from registers (not from the cache) by whoever owns position pos_new
  const T* kc = reinterpret_cast<const T*>(p.k_cur) + ((int64_t)b * p.Hkv + h) * D + sl * 8;
  const T* vc = reinterpret_cast<const T*>(p.v_cur) + ((int64_t)b * p.Hkv + h) * D + sl * 8;
  const uint4 kn = ld_stream16(kc), vn = ld_stream16(vc);
  if (s == 0 && warp == 0 && sub == 0) {
    T* krow = cache + base + (row0 + pos_new) * p.row_stride;
    *reinterpret_cast<uint4*>(krow) = kn;
    *reinterpret_cast<uint4*>(krow + p.kv_stride) = vn;
  }
  float m[kMaxGroup], l[kMaxGroup], acc[kMaxGroup][8];
#pragma unroll
  for (int g = 0; g < kMaxGroup; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int v = 0; v < 8; ++v) acc[g][v] = 0.f;
  }
  const int64_t p_begin = (int64_t)s * p.chunk;
  const int64_t p_end = min(kvlen, p_begin + p.chunk);
  // kUnroll load rounds per iteration: 2 x kUnroll 16-byte loads of every lane are in flight
  // before the first is used, and the dot products reduce as independent shuffle chains
  constexpr int kStep = PPL * kUnroll;          // positions of a warp per iteration
  for (int64_t pos0 = p_begin + (int64_t)warp * kStep; pos0 < p_end; pos0 += kAttnWarps * kStep) {
    uint4 kraw[kUnroll], vraw[kUnroll];
    bool valid[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t pos = pos0 + u * PPL + sub;
      valid[u] = pos < p_end;
      if (!valid[u]) {
        kraw[u] = make_uint4(0, 0, 0, 0);
        vraw[u] = kraw[u];
      } else if (pos == pos_new) {
        kraw[u] = kn;
        vraw[u] = vn;
      } else {
        const T* krow = cache + base + (row0 + pos) * p.row_stride;
        kraw[u] = __ldcg(reinterpret_cast<const uint4*>(krow));
        vraw[u] = __ldcg(reinterpret_cast<const uint4*>(krow + p.kv_stride));
      }
    }
    float kf[kUnroll][8];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) unpack16<T>(kraw[u], kf[u]);
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) {
      if (g < G) {
        float dot[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          dot[u] = 0.f;
#pragma unroll
          for (int v = 0; v < 8; ++v) dot[u] = fmaf(qv[g][v], kf[u][v], dot[u]);
        }
#pragma unroll
        for (int o = LPP / 2; o > 0; o >>= 1) {
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) dot[u] += __shfl_xor_sync(0xFFFFFFFFu, dot[u], o);
        }
        float m_new = m[g];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
          if (valid[u]) m_new = fmaxf(m_new, dot[u]);
        if (m_new == -INFINITY) continue;          // this lane group has seen no position yet
        const float corr = __expf(m[g] - m_new);
        float lsum = l[g] * corr;
#pragma unroll
        for (int v = 0; v < 8; ++v) acc[g][v] *= corr;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const float pr = valid[u] ? __expf(dot[u] - m_new) : 0.f;
          lsum += pr;
          float vf[8];
          unpack16<T>(vraw[u], vf);
#pragma unroll
          for (int v = 0; v < 8; ++v) acc[g][v] = fmaf(pr, vf[v], acc[g][v]);
        }
        l[g] = lsum;
        m[g] = m_new;
      }
    }
  }
  // merge the lane groups of the warp (same dims, different positions) ...
#pragma unroll
  for (int o = LPP; o < 32; o <<= 1) {
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) {
      if (g < G) {
        const float m_o = __shfl_xor_sync(0xFFFFFFFFu, m[g], o);
        const float l_o = __shfl_xor_sync(0xFFFFFFFFu, l[g], o);
        const float mm = fmaxf(m[g], m_o);
        const float c_me = m[g] == -INFINITY ? 0.f : __expf(m[g] - mm);
        const float c_o = m_o == -INFINITY ? 0.f : __expf(m_o - mm);
        l[g] = l[g] * c_me + l_o * c_o;
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          const float a_o = __shfl_xor_sync(0xFFFFFFFFu, acc[g][v], o);
          acc[g][v] = acc[g][v] * c_me + a_o * c_o;
        }
        m[g] = mm;
      }
    }
  }
  // ... and the warps of the CTA
#pragma unroll
  for (int g = 0; g < kMaxGroup; ++g) {
    if (g < G && sub == 0) {
#pragma unroll
      for (int v = 0; v < 8; ++v) sm_acc[warp][g][sl * 8 + v] = acc[g][v];
      if (sl == 0) {
        sm_m[warp][g] = m[g];
        sm_l[warp][g] = l[g];
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float c = sm_m[w][g] == -INFINITY ? 0.f : __expf(sm_m[w][g] - mm);
      ll += sm_l[w][g] * c;
      a += sm_acc[w][g][d] * c;
    }
    if (p.splits == 1) {
      reinterpret_cast<T*>(p.out)[((int64_t)b * p.Hq + (int64_t)h * G + g) * D + d] = Elem<T>::from_f(a / ll);
    } else {
      float* dst = p.part + ((((int64_t)b * p.Hkv + h) * p.splits + s) * G + g) * (D + 2);
      dst[d] = a;
      if (d == 0) {
        dst[D] = mm;
        dst[D + 1] = ll;
      }
    }
  }
}

// ---- tensor-core variant ---------------------------------------------------------
// The same work split, with the two small matrix products of a slice on the tensor cores
// (mma.sync m16n8k16, fp32 accumulation): S = Q K^T with the query heads of the group on
// MMA-M (padded to 16 rows) and 16 cached positions on MMA-N, O += P V with the head
// dimension on MMA-N.  The kernel needs 2 FLOP per cache byte, so the legacy tensor path
// is far from a limit; what it removes are the conversions and multiply-adds that kept
// the CUDA-core version instruction-bound.  Every warp owns a ring of kMmaStages tiles
// (16 positions x {keys, values}) in shared memory, filled with cp.async (16 bytes per
// lane, zero fill behind the end of the slice) and read with ldmatrix (values transposed);
// 16-byte chunks of a row are XOR-swizzled with the row index so that neither is bank
// conflicted.  The S accumulator fragments are the A fragments of P as they are.
constexpr int kMmaStages = 3;
constexpr int kMmaTile = 16;          // cached positions per tile

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  if constexpr (sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}
template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  } else {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(kAttnWarps * 32, 2)
decode_attention_mma_kernel(const AttnParams p) {
  constexpr int CH = D / 8;                       // 16-byte chunks per head row
  constexpr int ROWB = D * 2;                     // bytes per head row
  constexpr int TILEB = kMmaTile * ROWB;          // one tile of keys (or values)
  constexpr int KS = D / 16;                      // k-steps of Q K^T
  constexpr int NT = D / 8;                       // n-tiles of P V
  extern __shared__ __align__(128) uint8_t attn_smem[];
  __shared__ float sm_m[kAttnWarps][kGroupLimit], sm_l[kAttnWarps][kGroupLimit];
  const int b = blockIdx.x, h = blockIdx.y, s = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = p.Hq / p.Hkv;
  const int r = lane >> 2, cq = lane & 3;         // fragment row (query head of the group), column pair
  pdl_launch_dependents();
  pdl_wait();
  const int64_t pos_new = p.start_pos[b];
  const int64_t kvlen = pos_new + 1;
  const int64_t row0 = p.cachestarts[b];
  const T* cache = reinterpret_cast<const T*>(p.cache);
  const int64_t base = p.layer_off + (int64_t)h * p.head_stride;
  const T* kc = reinterpret_cast<const T*>(p.k_cur) + ((int64_t)b * p.Hkv + h) * D;
  const T* vc = reinterpret_cast<const T*>(p.v_cur) + ((int64_t)b * p.Hkv + h) * D;
  if (s == 0 && warp == 0 && lane < 2 * CH) {
    // the new key / value of this sequence and kv head go into the cache
    const int which = lane / CH, c = lane % CH;
    T* dst = reinterpret_cast<T*>(p.cache) + base + (row0 + pos_new) * p.row_stride + which * p.kv_stride + c * 8;
    *reinterpret_cast<uint4*>(dst) = ld_stream16((which ? vc : kc) + c * 8);
  }
  // A fragments of Q (rows >= G and rows 8..15 are zero)
  uint32_t qa[KS][2];
  {
    const T* q = reinterpret_cast<const T*>(p.q) + ((int64_t)b * p.Hq + (int64_t)h * G + r) * D;
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      qa[kk][0] = r < G ? *reinterpret_cast<const uint32_t*>(q + kk * 16 + cq * 2) : 0u;
      qa[kk][1] = r < G ? *reinterpret_cast<const uint32_t*>(q + kk * 16 + 8 + cq * 2) : 0u;
    }
  }
  float o[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m_run = -INFINITY, l_run = 0.f;           // of row r; l_run is this lane's share of the row sum

  const int64_t p_begin = (int64_t)s * p.chunk;
  const int64_t p_end = min(kvlen, p_begin + p.chunk);
  const int64_t n_pos = p_end > p_begin ? p_end - p_begin : 0;
  const int tiles_cta = (int)((n_pos + kMmaTile - 1) / kMmaTile);
  const int my_tiles = tiles_cta > warp ? (tiles_cta - warp + kAttnWarps - 1) / kAttnWarps : 0;
  const uint32_t ring = smem_u32_attn(attn_smem) + warp * (kMmaStages * 2 * TILEB);

  auto issue = [&](int i) {      // tile i of this warp -> stage i % kMmaStages
    const int64_t pos0 = p_begin + ((int64_t)warp + (int64_t)i * kAttnWarps) * kMmaTile;
    const uint32_t st = ring + (i % kMmaStages) * (2 * TILEB);
#pragma unroll
    for (int j = 0; j < kMmaTile * CH / 32; ++j) {
      const int c = lane + 32 * j;
      const int row = c / CH, ch = c % CH;
      const int64_t pos = pos0 + row;
      const uint32_t dst = st + row * ROWB + ((ch ^ (row & 7)) << 4);
      const bool valid = pos < p_end;
      const T* ksrc = pos == pos_new ? kc + ch * 8 : cache + base + (row0 + (valid ? pos : p_begin)) * p.row_stride + ch * 8;
      const T* vsrc = pos == pos_new ? vc + ch * 8 : ksrc + p.kv_stride;
      cp_async16(dst, ksrc, valid ? 16 : 0);
      cp_async16(dst + TILEB, vsrc, valid ? 16 : 0);
    }
  };
#pragma unroll
  for (int i = 0; i < kMmaStages - 1; ++i) {
    if (i < my_tiles) issue(i);
    cp_async_commit();
  }
  for (int i = 0; i < my_tiles; ++i) {
    cp_async_wait<kMmaStages - 2>();
    __syncwarp();                                   // tile i has landed; every lane is done with tile i - 1
    if (i + kMmaStages - 1 < my_tiles) issue(i + kMmaStages - 1);   // into the stage tile i - 1 used
    cp_async_commit();
    const int64_t pos0 = p_begin + ((int64_t)warp + (int64_t)i * kAttnWarps) * kMmaTile;
    const uint32_t st = ring + (i % kMmaStages) * (2 * TILEB);
    // S = Q K^T for the tile's 16 positions (two n-tiles of 8)
    float sc[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f; }
    {
      const int mi = lane >> 3;
      const int row = 8 * (mi >> 1) + (lane & 7);
#pragma unroll
      for (int kk = 0; kk < KS; ++kk) {
        uint32_t kb[4];
        const int ch = 2 * kk + (mi & 1);
        ldmatrix_x4(st + row * ROWB + ((ch ^ (row & 7)) << 4), kb);
        mma16816<T>(sc[0], qa[kk][0], 0u, qa[kk][1], 0u, kb[0], kb[1]);
        mma16816<T>(sc[1], qa[kk][0], 0u, qa[kk][1], 0u, kb[2], kb[3]);
      }
    }
    // online softmax of row r over the tile (this lane holds positions 8j + 2cq, +1)
    float pr[2][2];
    float tmax = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const bool valid = pos0 + 8 * j + 2 * cq + e < p_end;
        pr[j][e] = valid ? sc[j][e] * p.scale : -INFINITY;
        tmax = fmaxf(tmax, pr[j][e]);
      }
    }
    tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFu, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFu, tmax, 2));
    const float m_new = fmaxf(m_run, tmax);        // finite: every tile holds at least one position
    const float corr = __expf(m_run - m_new);
    float psum = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        pr[j][e] = __expf(pr[j][e] - m_new);
        psum += pr[j][e];
      }
    }
    l_run = l_run * corr + psum;
    m_run = m_new;
#pragma unroll
    for (int j = 0; j < NT; ++j) { o[j][0] *= corr; o[j][1] *= corr; }
    // O += P V: the S fragments are the A fragments of P (rows of padding stay zero)
    const uint32_t pa0 = r < G ? pack2<T>(pr[0][0], pr[0][1]) : 0u;
    const uint32_t pa2 = r < G ? pack2<T>(pr[1][0], pr[1][1]) : 0u;
    {
      const int mi = lane >> 3;
      const int row = 8 * (mi & 1) + (lane & 7);
#pragma unroll
      for (int jn = 0; jn < NT; jn += 2) {
        uint32_t vb[4];
        const int ch = jn + (mi >> 1);
        ldmatrix_x4_trans(st + TILEB + row * ROWB + ((ch ^ (row & 7)) << 4), vb);
        mma16816<T>(o[jn], pa0, 0u, pa2, 0u, vb[0], vb[1]);
        mma16816<T>(o[jn + 1], pa0, 0u, pa2, 0u, vb[2], vb[3]);
      }
    }
  }
  cp_async_wait<0>();
  // the row sum of this warp, then the warps of the CTA meet in shared memory (the ring is free now)
  l_run += __shfl_xor_sync(0xFFFFFFFFu, l_run, 1);
  l_run += __shfl_xor_sync(0xFFFFFFFFu, l_run, 2);
  __syncthreads();
  float* sm_acc = reinterpret_cast<float*>(attn_smem);          // [warps][kGroupLimit][D]
  if (r < G) {
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      float* dst = sm_acc + ((size_t)warp * kGroupLimit + r) * D + 8 * j + 2 * cq;
      dst[0] = o[j][0];
      dst[1] = o[j][1];
    }
    if (cq == 0) {
      sm_m[warp][r] = m_run;
      sm_l[warp][r] = l_run;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float c = sm_m[w][g] == -INFINITY ? 0.f : __expf(sm_m[w][g] - mm);
      ll += sm_l[w][g] * c;
      a += sm_acc[((size_t)w * kGroupLimit + g) * D + d] * c;
    }
    if (p.splits == 1) {
      reinterpret_cast<T*>(p.out)[((int64_t)b * p.Hq + (int64_t)h * G + g) * D + d] = Elem<T>::from_f(a / ll);
    } else {
      float* dst = p.part + ((((int64_t)b * p.Hkv + h) * p.splits + s) * G + g) * (D + 2);
      dst[d] = a;
      if (d == 0) {
        dst[D] = mm;
        dst[D + 1] = ll;
      }
    }
  }
}

// out[b, head, :] = sum over slices of acc * exp(max - global max) / sum of the same for l
template <typename T>
__global__ void decode_attention_merge_kernel(const float* part, T* __restrict__ out, int Hq, int Hkv,
                                              int splits, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, head = blockIdx.y;
  const int G = Hq / Hkv, h = head / G, g = head - h * G;
  const float* base = part + ((((int64_t)b * Hkv + h) * splits) * G + g) * (D + 2);
  const int64_t stride = (int64_t)G * (D + 2);
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, base[s * stride + D]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f, ll = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = base[s * stride + D];
      const float c = ms == -INFINITY ? 0.f : __expf(ms - mm);
      a += base[s * stride + d] * c;
      ll += base[s * stride + D + 1] * c;
    }
    out[((int64_t)b * Hq + head) * D + d] = Elem<T>::from_f(a / ll);
  }
}

std::atomic<int> g_variant{0};   // 0: tensor-core kernel, 1: CUDA-core kernel

int pick_splits(int64_t B, int Hkv, int64_t max_kvlen, int variant) {
  // CUDA-core kernel: enough CTAs for twelve 4-warp CTAs per SM (it hides latency with warps,
  // not with bytes in flight per warp), slices of at least 64 positions.  Tensor-core kernel:
  // two CTAs per SM with a ring of tiles per warp; three waves, at least four tiles per warp.
  const int64_t want = ceil_div((variant == 1 ? 12 : 6) * (int64_t)sm_count(), B * Hkv);
  int64_t cap = ceil_div(max_kvlen, variant == 1 ? 64 : 4 * kAttnWarps * kMmaTile);
  int64_t s = want < cap ? want : cap;
  if (s < 1) s = 1;
  if (s > 64) s = 64;
  return (int)s;
}

}  // namespace

int decode_attention_set_variant(int variant) {
  return g_variant.exchange(variant == 1 ? 1 : 0, std::memory_order_relaxed);
}

size_t decode_attention_workspace_bytes(int64_t B, int Hq, int Hkv, int D, int64_t max_kvlen) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || max_kvlen <= 0) return 0;
  const int a = pick_splits(B, Hkv, max_kvlen, 0), b = pick_splits(B, Hkv, max_kvlen, 1);
  return 256 + (size_t)B * Hq * (a > b ? a : b) * (D + 2) * sizeof(float);
}

int launch_decode_attention(const void* q, const void* k_cur, const void* v_cur, void* cache,
                            const int64_t* cachestarts, const int64_t* start_pos, void* out, int64_t B, int Hq,
                            int Hkv, int D, int64_t layer_off, int64_t row_stride, int64_t kv_stride,
                            int64_t head_stride, int64_t max_kvlen, int dtype, void* ws, size_t ws_bytes,
                            cudaStream_t s) {
  if (!q || !k_cur || !v_cur || !cache || !cachestarts || !start_pos || !out)
    return fail(PMX_ERR_INVALID_ARGUMENT, "decode_cache_attention: null pointer");
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || max_kvlen <= 0 || Hq % Hkv)
    return fail(PMX_ERR_INVALID_ARGUMENT, "decode_cache_attention: B, heads and max_kvlen must be positive and num_heads a multiple of num_kv_heads (B=%lld Hq=%d Hkv=%d)", (long long)B, Hq, Hkv);
  if (Hq / Hkv > kGroupLimit)
    return fail(PMX_ERR_UNSUPPORTED, "decode_cache_attention: at most %d query heads per key/value head", kGroupLimit);
  if (D != 64 && D != 128) return fail(PMX_ERR_UNSUPPORTED, "decode_cache_attention: head_dim %d (64 and 128 are covered)", D);
  if (dtype != PMX_DTYPE_F16 && dtype != PMX_DTYPE_BF16)
    return fail(PMX_ERR_UNSUPPORTED, "decode_cache_attention: float16 and bfloat16 caches are covered");
  if (B > 65535 * 32ll) return fail(PMX_ERR_UNSUPPORTED, "decode_cache_attention: too many sequences");
  if (row_stride % 8 || kv_stride % 8 || head_stride % 8 || layer_off % 8 || !aligned16(cache) || !aligned16(q) ||
      !aligned16(k_cur) || !aligned16(v_cur))
    return fail(PMX_ERR_ALIGNMENT, "decode_cache_attention: tensors and cache strides must keep head rows 16-byte aligned");
  const size_t need = decode_attention_workspace_bytes(B, Hq, Hkv, D, max_kvlen);
  if (!ws || ws_bytes < need) return fail(PMX_ERR_WORKSPACE, "decode_cache_attention: workspace of %zu bytes needed, %zu given", need, ws_bytes);
  AttnParams p{};
  p.q = q; p.k_cur = k_cur; p.v_cur = v_cur; p.cache = cache;
  p.cachestarts = cachestarts; p.start_pos = start_pos; p.out = out;
  p.part = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + 256);
  p.layer_off = layer_off; p.row_stride = row_stride; p.kv_stride = kv_stride; p.head_stride = head_stride;
  p.B = (int)B; p.Hq = Hq; p.Hkv = Hkv;
  const int variant = g_variant.load(std::memory_order_relaxed);
  p.splits = pick_splits(B, Hkv, max_kvlen, variant);
  p.chunk = (int)ceil_div(max_kvlen, p.splits);
  p.scale = 1.0f / sqrtf((float)D);
  const dim3 grid((unsigned)B, (unsigned)Hkv, (unsigned)p.splits);
  const bool bf = dtype == PMX_DTYPE_BF16;
  const int G = Hq / Hkv;
  const void* kern = nullptr;
#define PMX_ATTN_PICK(GM)                                                                                         \
  kern = D == 128 ? (bf ? (const void*)decode_attention_kernel<__nv_bfloat16, 128, GM>                            \
                        : (const void*)decode_attention_kernel<__half, 128, GM>)                                   \
                  : (bf ? (const void*)decode_attention_kernel<__nv_bfloat16, 64, GM>                             \
                        : (const void*)decode_attention_kernel<__half, 64, GM>)
  if (G == 1) { PMX_ATTN_PICK(1); } else if (G == 2) { PMX_ATTN_PICK(2); } else if (G <= 4) { PMX_ATTN_PICK(4); } else { PMX_ATTN_PICK(8); }
#undef PMX_ATTN_PICK
  size_t smem = 0;
  if (variant == 0) {
    kern = D == 128 ? (bf ? (const void*)decode_attention_mma_kernel<__nv_bfloat16, 128>
                          : (const void*)decode_attention_mma_kernel<__half, 128>)
                    : (bf ? (const void*)decode_attention_mma_kernel<__nv_bfloat16, 64>
                          : (const void*)decode_attention_mma_kernel<__half, 64>);
    smem = (size_t)kAttnWarps * kMmaStages * 2 * kMmaTile * D * 2;
    PMX_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  void* args[] = {(void*)&p};
  int st = launch_pdl(kern, grid, dim3(kAttnWarps * 32), smem, s, args);
  if (st != PMX_OK || p.splits == 1) return st;
  const dim3 mgrid((unsigned)B, (unsigned)Hq);
  if (bf)
    return launch_pdl_k(decode_attention_merge_kernel<__nv_bfloat16>, mgrid, dim3(D), 0, s, (const float*)p.part,
                        (__nv_bfloat16*)out, Hq, Hkv, p.splits, D);
  return launch_pdl_k(decode_attention_merge_kernel<__half>, mgrid, dim3(D), 0, s, (const float*)p.part, (__half*)out,
                      Hq, Hkv, p.splits, D);
}

}  // namespace pmx
