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
#include "common.cuh"

namespace pmx {
namespace {

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

int pick_splits(int64_t B, int Hkv, int64_t max_kvlen) {
  // enough CTAs for twelve 4-warp CTAs per SM (the kernel hides latency with warps, not
  // with bytes in flight per warp), slices of at least 64 positions
  const int64_t want = ceil_div(12 * (int64_t)sm_count(), B * Hkv);
  int64_t cap = ceil_div(max_kvlen, 64);
  int64_t s = want < cap ? want : cap;
  if (s < 1) s = 1;
  if (s > 64) s = 64;
  return (int)s;
}

}  // namespace

size_t decode_attention_workspace_bytes(int64_t B, int Hq, int Hkv, int D, int64_t max_kvlen) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || max_kvlen <= 0) return 0;
  const int splits = pick_splits(B, Hkv, max_kvlen);
  return 256 + (size_t)B * Hq * splits * (D + 2) * sizeof(float);
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
  p.splits = pick_splits(B, Hkv, max_kvlen);
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
  void* args[] = {(void*)&p};
  int st = launch_pdl(kern, grid, dim3(kAttnWarps * 32), 0, s, args);
  if (st != PMX_OK || p.splits == 1) return st;
  const dim3 mgrid((unsigned)B, (unsigned)Hq);
  if (bf)
    return launch_pdl_k(decode_attention_merge_kernel<__nv_bfloat16>, mgrid, dim3(D), 0, s, (const float*)p.part,
                        (__nv_bfloat16*)out, Hq, Hkv, p.splits, D);
  return launch_pdl_k(decode_attention_merge_kernel<__half>, mgrid, dim3(D), 0, s, (const float*)p.part, (__half*)out,
                      Hq, Hkv, p.splits, D);
}

}  // namespace pmx
