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
// query heads that share the kv head, one position per warp at a time (a 256-byte row is one
// coalesced load of the warp), with the running maximum / sum / weighted value sum of an
// online softmax in registers.  The slices of a (sequence, kv head) are merged by a second,
// tiny kernel.  All cache layouts of cache_mode 0 are covered through strides.
#include "common.cuh"

namespace pmx {
namespace {

constexpr int kAttnWarps = 4;
constexpr int kMaxGroup = 8;       // query heads per kv head

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

template <typename T, int VPL>   // VPL = head_dim / 32 values per lane
__global__ void __launch_bounds__(kAttnWarps * 32)
decode_attention_kernel(const AttnParams p) {
  constexpr int D = VPL * 32;
  const int b = blockIdx.x, h = blockIdx.y, s = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
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
  const int64_t base = p.layer_off + (int64_t)h * p.head_stride;

  // this lane's VPL dims of every query of the group, pre-scaled
  float qv[kMaxGroup][VPL];
#pragma unroll
  for (int g = 0; g < kMaxGroup; ++g) {
    if (g < G) {
#pragma unroll
      for (int v = 0; v < VPL; ++v) qv[g][v] = Elem<T>::to_f(q[(int64_t)g * D + lane * VPL + v]) * p.scale;
    }
  }
  // the new key / value of this sequence and kv head: stored into the cache by the CTA of
  // slice 0 and taken from registers (not from the cache) by whoever owns position pos_new
  float kn[VPL], vn[VPL];
  {
    const T* kc = reinterpret_cast<const T*>(p.k_cur) + ((int64_t)b * p.Hkv + h) * D + lane * VPL;
    const T* vc = reinterpret_cast<const T*>(p.v_cur) + ((int64_t)b * p.Hkv + h) * D + lane * VPL;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      kn[v] = Elem<T>::to_f(kc[v]);
      vn[v] = Elem<T>::to_f(vc[v]);
    }
    if (s == 0 && warp == 0) {
      T* krow = cache + base + (row0 + pos_new) * p.row_stride + lane * VPL;
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        krow[v] = kc[v];
        krow[p.kv_stride + v] = vc[v];
      }
    }
  }
  float m[kMaxGroup], l[kMaxGroup], acc[kMaxGroup][VPL];
#pragma unroll
  for (int g = 0; g < kMaxGroup; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v) acc[g][v] = 0.f;
  }
  const int64_t p_begin = (int64_t)s * p.chunk;
  const int64_t p_end = min(kvlen, p_begin + p.chunk);
  for (int64_t pos = p_begin + warp; pos < p_end; pos += kAttnWarps) {
    float kf[VPL], vf[VPL];
    if (pos == pos_new) {
#pragma unroll
      for (int v = 0; v < VPL; ++v) { kf[v] = kn[v]; vf[v] = vn[v]; }
    } else {
      const T* krow = cache + base + (row0 + pos) * p.row_stride + lane * VPL;
      // VPL 16-bit (or 32-bit) values per lane: one 8- or 16-byte load
      T kraw[VPL], vraw[VPL];
      if (sizeof(T) * VPL == 8) {
        *reinterpret_cast<uint2*>(kraw) = __ldg(reinterpret_cast<const uint2*>(krow));
        *reinterpret_cast<uint2*>(vraw) = __ldg(reinterpret_cast<const uint2*>(krow + p.kv_stride));
      } else if (sizeof(T) * VPL == 16) {
        *reinterpret_cast<uint4*>(kraw) = __ldg(reinterpret_cast<const uint4*>(krow));
        *reinterpret_cast<uint4*>(vraw) = __ldg(reinterpret_cast<const uint4*>(krow + p.kv_stride));
      } else {
#pragma unroll
        for (int v = 0; v < VPL; ++v) { kraw[v] = krow[v]; vraw[v] = krow[p.kv_stride + v]; }
      }
#pragma unroll
      for (int v = 0; v < VPL; ++v) { kf[v] = Elem<T>::to_f(kraw[v]); vf[v] = Elem<T>::to_f(vraw[v]); }
    }
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) {
      if (g < G) {
        float dot = 0.f;
#pragma unroll
        for (int v = 0; v < VPL; ++v) dot = fmaf(qv[g][v], kf[v], dot);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xFFFFFFFFu, dot, o);
        const float m_new = fmaxf(m[g], dot);
        const float corr = __expf(m[g] - m_new);
        const float pr = __expf(dot - m_new);
        l[g] = l[g] * corr + pr;
#pragma unroll
        for (int v = 0; v < VPL; ++v) acc[g][v] = fmaf(pr, vf[v], acc[g][v] * corr);
        m[g] = m_new;
      }
    }
  }
  // merge the warps of the CTA
#pragma unroll
  for (int g = 0; g < kMaxGroup; ++g) {
    if (g < G) {
#pragma unroll
      for (int v = 0; v < VPL; ++v) sm_acc[warp][g][lane * VPL + v] = acc[g][v];
      if (lane == 0) {
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
__global__ void decode_attention_merge_kernel(const float* __restrict__ part, T* __restrict__ out, int Hq, int Hkv,
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
  // enough CTAs to cover the SMs about three times, slices of at least 64 positions
  const int64_t want = ceil_div(3 * (int64_t)sm_count(), B * Hkv);
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
  if (Hq / Hkv > kMaxGroup)
    return fail(PMX_ERR_UNSUPPORTED, "decode_cache_attention: at most %d query heads per key/value head", kMaxGroup);
  if (D != 64 && D != 128) return fail(PMX_ERR_UNSUPPORTED, "decode_cache_attention: head_dim %d (64 and 128 are covered)", D);
  if (dtype != PMX_DTYPE_F16 && dtype != PMX_DTYPE_BF16)
    return fail(PMX_ERR_UNSUPPORTED, "decode_cache_attention: float16 and bfloat16 caches are covered");
  if (B > 65535 * 32ll) return fail(PMX_ERR_UNSUPPORTED, "decode_cache_attention: too many sequences");
  const int vpl = D / 32;
  if (row_stride % vpl || kv_stride % vpl || head_stride % vpl || layer_off % vpl || !aligned16(cache) || !aligned16(q))
    return fail(PMX_ERR_ALIGNMENT, "decode_cache_attention: cache strides must keep head rows %d-byte aligned", vpl * 2);
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
  int st;
  const bool bf = dtype == PMX_DTYPE_BF16;
  if (D == 128)
    st = bf ? launch_pdl_k(decode_attention_kernel<__nv_bfloat16, 4>, grid, dim3(kAttnWarps * 32), 0, s, p)
            : launch_pdl_k(decode_attention_kernel<__half, 4>, grid, dim3(kAttnWarps * 32), 0, s, p);
  else
    st = bf ? launch_pdl_k(decode_attention_kernel<__nv_bfloat16, 2>, grid, dim3(kAttnWarps * 32), 0, s, p)
            : launch_pdl_k(decode_attention_kernel<__half, 2>, grid, dim3(kAttnWarps * 32), 0, s, p);
  if (st != PMX_OK || p.splits == 1) return st;
  const dim3 mgrid((unsigned)B, (unsigned)Hq);
  if (bf)
    return launch_pdl_k(decode_attention_merge_kernel<__nv_bfloat16>, mgrid, dim3(D), 0, s, (const float*)p.part,
                        (__nv_bfloat16*)out, Hq, Hkv, p.splits, D);
  return launch_pdl_k(decode_attention_merge_kernel<__half>, mgrid, dim3(D), 0, s, (const float*)p.part, (__half*)out,
                      Hq, Hkv, p.splits, D);
}

}  // namespace pmx
