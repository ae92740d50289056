// HBM-bound kernels around the expert GEMMs: the top-k weighted combine
// (moe_reduce), the stand-alone SwiGLU / SiLU activations, the zero fill of
// rows no expert owns and the final sum of split-K partial results.
// All of them move 16 bytes per thread access and accumulate in fp32.
#include "common.cuh"

namespace pmx {
namespace {

constexpr int kThreads = 256;

inline int grid_for(int64_t work_items) {
  int64_t blocks = ceil_div(work_items, kThreads);
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

// out[t,:] = sum_j w[t,j] * y[inv[t,j],:]      (MoeReduce.py:23-25)
// One thread produces 16 bytes of one output row.  The rows of up to 4 slots are
// requested together so that their HBM latencies overlap.
template <typename T, bool VEC>
__device__ __forceinline__ void reduce_item(const T* y, const T* w,
                                            const int64_t* inv, T* __restrict__ out,
                                            int k, int64_t N, int64_t chunks, int64_t i) {
  constexpr int V = VEC ? kVec<T> : 1;
  const int64_t t = i / chunks, c = i - t * chunks;
  float acc[V];
#pragma unroll
  for (int v = 0; v < V; ++v) acc[v] = 0.f;
  if (VEC) {
    for (int j0 = 0; j0 < k; j0 += 4) {
      uint4 raw[4];
      float wj[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j0 + j < k) {
          const int64_t r = inv[t * k + j0 + j];
          wj[j] = Elem<T>::to_f(w[t * k + j0 + j]);
          raw[j] = ld_stream16(y + r * N + c * V);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j0 + j < k) {
          float f[kVec<T>];
          unpack16<T>(raw[j], f);
#pragma unroll
          for (int v = 0; v < V; ++v) acc[v] = fmaf(wj[j], f[v], acc[v]);
        }
      }
    }
    float f[kVec<T>];
#pragma unroll
    for (int v = 0; v < V; ++v) f[v] = acc[v];
    *reinterpret_cast<uint4*>(out + t * N + c * V) = pack16<T>(f);
  } else {
    for (int j = 0; j < k; ++j) {
      const int64_t r = inv[t * k + j];
      acc[0] = fmaf(Elem<T>::to_f(w[t * k + j]), Elem<T>::to_f(y[r * N + c]), acc[0]);
    }
    out[t * N + c] = Elem<T>::from_f(acc[0]);
  }
}

template <typename T, bool VEC>
__global__ void reduce_kernel(const T* y, const T* w,
                              const int64_t* inv, T* __restrict__ out, int64_t Tn,
                              int k, int64_t N) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = VEC ? kVec<T> : 1;
  const int64_t chunks = N / V;
  const int64_t total = Tn * chunks;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  // (two items per iteration were measured slower on B200: 58 us against 45 us for
  // the 8192-token bf16 combine, the extra registers cost more occupancy than the
  // overlap gains)
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
    reduce_item<T, VEC>(y, w, inv, out, k, N, chunks, i);
}

// y[m, j] = x[m, D/2 + j] * x[m, j] * sigmoid(beta * x[m, j])    (SwiGLU.py:15-16)
template <typename T, bool VEC>
__global__ void swiglu_kernel(const T* x, T* __restrict__ y, int64_t M, int64_t D,
                              float beta) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = VEC ? kVec<T> : 1;
  const int64_t half = D / 2, chunks = half / V, total = M * chunks;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / chunks, c = i - m * chunks;
    if (VEC) {
      float a[kVec<T>], g[kVec<T>];
      unpack16<T>(ld_stream16(x + m * D + c * V), a);
      unpack16<T>(ld_stream16(x + m * D + half + c * V), g);
#pragma unroll
      for (int v = 0; v < V; ++v) a[v] = g[v] * a[v] / (1.0f + expf(-beta * a[v]));
      *reinterpret_cast<uint4*>(y + m * half + c * V) = pack16<T>(a);
    } else {
      const float a = Elem<T>::to_f(x[m * D + c]), g = Elem<T>::to_f(x[m * D + half + c]);
      y[m * half + c] = Elem<T>::from_f(g * a / (1.0f + expf(-beta * a)));
    }
  }
}

// y = silu(x) (* gate)    (SiLU.py:18-21)
template <typename T, bool VEC>
__global__ void silu_kernel(const T* x, const T* gate, T* __restrict__ y,
                            int64_t n) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = VEC ? kVec<T> : 1;
  const int64_t total = n / V;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    if (VEC) {
      float a[kVec<T>], g[kVec<T>];
      unpack16<T>(ld_stream16(x + i * V), a);
      if (gate) unpack16<T>(ld_stream16(gate + i * V), g);
#pragma unroll
      for (int v = 0; v < V; ++v) {
        a[v] = a[v] / (1.0f + expf(-a[v]));
        if (gate) a[v] *= g[v];
      }
      *reinterpret_cast<uint4*>(y + i * V) = pack16<T>(a);
    } else {
      float a = Elem<T>::to_f(x[i]);
      a = a / (1.0f + expf(-a));
      if (gate) a *= Elem<T>::to_f(gate[i]);
      y[i] = Elem<T>::from_f(a);
    }
  }
}

// RMSNorm with an optional skip connection (RMSNorm.py:15-24 and :42-56):
//   s = x (+ skip), rounded to T;  y = T(float(s) * rsqrt(mean(s^2) + eps)) * weight
// One block per row.  Rows of up to 4 x 256 sixteen-byte chunks (8192 halves) stay in
// registers between the sum of squares and the scaling (REG); longer or unaligned
// rows are read a second time (from L1/L2).  The two roundings of the reference
// (`Y.type_as(X) * weight`) are reproduced.
__device__ __forceinline__ float block_sum_256(float acc, float* warp_sums, float* result) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += warp_sums[w];
    *result = tot;
  }
  __syncthreads();
  return *result;
}

template <typename T, bool VEC, bool REG>
__global__ void __launch_bounds__(256)
skip_rms_norm_kernel(const T* x, const T* skip, const T* weight,
                     T* __restrict__ y, T* __restrict__ skip_out, int64_t M, int64_t H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = VEC ? kVec<T> : 1;
  constexpr int R = 4;   // chunks per thread held in registers (REG)
  __shared__ float warp_sums[8];
  __shared__ float s_total;
  const int64_t chunks = H / V;
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const T* xr = x + row * H;
    const T* sr = skip ? skip + row * H : nullptr;
    T* so = skip_out + row * H;
    float acc = 0.f;
    if (REG) {
      float a[R][kVec<T>];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int64_t c = threadIdx.x + (int64_t)r * blockDim.x;
        if (c < chunks) {
          unpack16<T>(ld_stream16(xr + c * kVec<T>), a[r]);
          if (sr) {
            float b[kVec<T>];
            unpack16<T>(ld_stream16(sr + c * kVec<T>), b);
#pragma unroll
            for (int v = 0; v < kVec<T>; ++v) a[r][v] = Elem<T>::to_f(Elem<T>::from_f(a[r][v] + b[v]));
            *reinterpret_cast<uint4*>(so + c * kVec<T>) = pack16<T>(a[r]);
          }
#pragma unroll
          for (int v = 0; v < kVec<T>; ++v) acc = fmaf(a[r][v], a[r][v], acc);
        }
      }
      const float scale = rsqrtf(block_sum_256(acc, warp_sums, &s_total) / (float)H + eps);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int64_t c = threadIdx.x + (int64_t)r * blockDim.x;
        if (c < chunks) {
          float wv[kVec<T>];
          unpack16<T>(ld_nc16(weight + c * kVec<T>), wv);
#pragma unroll
          for (int v = 0; v < kVec<T>; ++v) a[r][v] = Elem<T>::to_f(Elem<T>::from_f(a[r][v] * scale)) * wv[v];
          *reinterpret_cast<uint4*>(y + row * H + c * kVec<T>) = pack16<T>(a[r]);
        }
      }
      __syncthreads();
      continue;
    }
    for (int64_t c = threadIdx.x; c < chunks; c += blockDim.x) {
      if (VEC) {
        float a[kVec<T>], b[kVec<T>];
        unpack16<T>(ld_stream16(xr + c * V), a);
        if (sr) {
          unpack16<T>(ld_stream16(sr + c * V), b);
#pragma unroll
          for (int v = 0; v < V; ++v) a[v] = Elem<T>::to_f(Elem<T>::from_f(a[v] + b[v]));
          *reinterpret_cast<uint4*>(so + c * V) = pack16<T>(a);
        }
#pragma unroll
        for (int v = 0; v < V; ++v) acc = fmaf(a[v], a[v], acc);
      } else {
        float a = Elem<T>::to_f(xr[c]);
        if (sr) {
          a = Elem<T>::to_f(Elem<T>::from_f(a + Elem<T>::to_f(sr[c])));
          so[c] = Elem<T>::from_f(a);
        }
        acc = fmaf(a, a, acc);
      }
    }
    const float scale = rsqrtf(block_sum_256(acc, warp_sums, &s_total) / (float)H + eps);
    const T* src = sr ? so : xr;      // the rounded sum written above, or x itself
    for (int64_t c = threadIdx.x; c < chunks; c += blockDim.x) {
      if (VEC) {
        float a[kVec<T>], wv[kVec<T>];
        unpack16<T>(*reinterpret_cast<const uint4*>(src + c * V), a);
        unpack16<T>(ld_nc16(weight + c * V), wv);
#pragma unroll
        for (int v = 0; v < V; ++v) a[v] = Elem<T>::to_f(Elem<T>::from_f(a[v] * scale)) * wv[v];
        *reinterpret_cast<uint4*>(y + row * H + c * V) = pack16<T>(a);
      } else {
        const float a = Elem<T>::to_f(Elem<T>::from_f(Elem<T>::to_f(src[c]) * scale));
        y[row * H + c] = Elem<T>::from_f(a * Elem<T>::to_f(weight[c]));
      }
    }
    __syncthreads();
  }
}

// Many rows (prefill): a WARP per row, the whole row (up to 16 sixteen-byte chunks per lane, kept
// as the rounded T values) in registers, no block-wide barrier: all of a row's loads are in
// flight at once and the reduction is five shuffles.
template <typename T>
__global__ void __launch_bounds__(256)
skip_rms_norm_warp_kernel(const T* x, const T* skip, const T* weight,
                          T* __restrict__ y, T* __restrict__ skip_out, int64_t M, int64_t H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = kVec<T>;
  constexpr int R = 16;                       // chunks per lane
  const int lane = threadIdx.x & 31;
  const int chunks = (int)(H / V);
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < M; row += warps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
    const uint4* sr = skip ? reinterpret_cast<const uint4*>(skip + row * H) : nullptr;
    uint4 a[R], b[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int c = lane + 32 * r;
      if (c < chunks) {
        a[r] = __ldcg(xr + c);
        if (sr) b[r] = __ldcg(sr + c);
      }
    }
    float acc = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int c = lane + 32 * r;
      if (c < chunks) {
        float f[V];
        unpack16<T>(a[r], f);
        if (sr) {
          float g[V];
          unpack16<T>(b[r], g);
#pragma unroll
          for (int v = 0; v < V; ++v) f[v] = Elem<T>::to_f(Elem<T>::from_f(f[v] + g[v]));
          a[r] = pack16<T>(f);
          reinterpret_cast<uint4*>(skip_out + row * H)[c] = a[r];
        }
#pragma unroll
        for (int v = 0; v < V; ++v) acc = fmaf(f[v], f[v], acc);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    const float scale = rsqrtf(acc / (float)H + eps);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int c = lane + 32 * r;
      if (c < chunks) {
        float f[V], wv[V];
        unpack16<T>(a[r], f);
        unpack16<T>(__ldg(reinterpret_cast<const uint4*>(weight) + c), wv);
#pragma unroll
        for (int v = 0; v < V; ++v) f[v] = Elem<T>::to_f(Elem<T>::from_f(f[v] * scale)) * wv[v];
        reinterpret_cast<uint4*>(y + row * H)[c] = pack16<T>(f);
      }
    }
  }
}

// rows outside [off[0], off[E]) <- 0   (the zero-initialised output of
// MoeColumnParallelLinear.py:59 / MoeRowParallelLinear.py:45)
template <typename T>
__global__ void zero_outside_kernel(T* __restrict__ y, const int64_t* off, int64_t M,
                                    int64_t n_out, int E) {
  pdl_launch_dependents();
  pdl_wait();
  int64_t lo = off[0], hi = off[E];
  lo = lo < 0 ? 0 : (lo > M ? M : lo);
  hi = hi < lo ? lo : (hi > M ? M : hi);
  const int64_t head = lo * n_out, tail = (M - hi) * n_out;
  const T zero = Elem<T>::from_f(0.f);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < head + tail;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t idx = i < head ? i : hi * n_out + (i - head);
    y[idx] = zero;
  }
}

// y[m,:] = cast(sum_s partial[s][m][:] (+ bias[e(m)])); rows no expert owns <- 0.
// With SWIGLU the partial rows hold [gate | up] (n_in = 2*n_out columns) and the
// activation is applied to the finished sums: y = up * gate * sigmoid(beta*gate).
template <typename T, bool SWIGLU>
__global__ void splitk_finish_kernel(const float* partial,
                                     const int64_t* off, const T* bias,
                                     T* __restrict__ y, int64_t M, int64_t n_out, int E, int split,
                                     float beta) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t n_in = SWIGLU ? 2 * n_out : n_out;
  const int64_t chunks = n_out / 4, total = M * chunks;
  const int64_t lo = offset_at(off, 0, M), hi = offset_at(off, E, M);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / chunks, c = (i - m * chunks) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f), up = make_float4(0.f, 0.f, 0.f, 0.f);
    if (m >= lo && m < hi) {
      for (int s = 0; s < split; ++s) {
        const float* row = partial + ((int64_t)s * M + m) * n_in;
        const float4 p = *reinterpret_cast<const float4*>(row + c);
        acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
        if (SWIGLU) {
          const float4 q = *reinterpret_cast<const float4*>(row + n_out + c);
          up.x += q.x; up.y += q.y; up.z += q.z; up.w += q.w;
        }
      }
      if (bias) {
        int e = 0;
        while (e + 1 < E && offset_at(off, e + 1, M) <= m) ++e;
        const T* b = bias + (int64_t)e * n_in + c;
        acc.x += Elem<T>::to_f(b[0]); acc.y += Elem<T>::to_f(b[1]);
        acc.z += Elem<T>::to_f(b[2]); acc.w += Elem<T>::to_f(b[3]);
        if (SWIGLU) {
          up.x += Elem<T>::to_f(b[n_out]); up.y += Elem<T>::to_f(b[n_out + 1]);
          up.z += Elem<T>::to_f(b[n_out + 2]); up.w += Elem<T>::to_f(b[n_out + 3]);
        }
      }
      if (SWIGLU) {
        acc.x = swiglu_f(acc.x, up.x, beta); acc.y = swiglu_f(acc.y, up.y, beta);
        acc.z = swiglu_f(acc.z, up.z, beta); acc.w = swiglu_f(acc.w, up.w, beta);
      }
    }
    T* o = y + m * n_out + c;
    o[0] = Elem<T>::from_f(acc.x); o[1] = Elem<T>::from_f(acc.y);
    o[2] = Elem<T>::from_f(acc.z); o[3] = Elem<T>::from_f(acc.w);
  }
}

// launch with programmatic stream serialisation (the kernels above wait for their
// predecessors first thing); counts the launch and returns on error
#define PMX_PDL_LAUNCH(kern, grid, block, smem, s, ...)                                        \
  do {                                                                                         \
    const int _st = launch_pdl_k(kern, dim3(grid), dim3(block), smem, s, __VA_ARGS__);         \
    if (_st != PMX_OK) return _st;                                                             \
  } while (0)

#define PMX_DISPATCH_DTYPE(dtype, what, ...)                                       \
  switch (dtype) {                                                                 \
    case PMX_DTYPE_F16: { using T = __half; __VA_ARGS__ } break;                   \
    case PMX_DTYPE_BF16: { using T = __nv_bfloat16; __VA_ARGS__ } break;           \
    case PMX_DTYPE_F32: { using T = float; __VA_ARGS__ } break;                    \
    default: return fail(PMX_ERR_UNSUPPORTED, what ": unknown dtype %d", dtype);   \
  }

}  // namespace

int launch_reduce(const void* y, const void* w, const int64_t* inv, void* out, int64_t Tn, int k,
                  int64_t N, int dtype, cudaStream_t s) {
  if (!y || !w || !inv || !out) return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce: null pointer");
  if (Tn <= 0 || k <= 0 || N <= 0) return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce: T, k, N must be positive");
  PMX_DISPATCH_DTYPE(dtype, "moe_reduce", {
    const bool vec = N % kVec<T> == 0 && aligned16(y) && aligned16(out);
    const int64_t items = Tn * (vec ? N / kVec<T> : N);
    if (vec)
      PMX_PDL_LAUNCH((reduce_kernel<T, true>), grid_for(items), kThreads, 0, s, (const T*)y, (const T*)w, inv, (T*)out, Tn, k, N);
    else
      PMX_PDL_LAUNCH((reduce_kernel<T, false>), grid_for(items), kThreads, 0, s, (const T*)y, (const T*)w, inv, (T*)out, Tn, k, N);
  })
  return PMX_OK;
}

int launch_swiglu(const void* x, void* y, int64_t M, int64_t D, float beta, int dtype, cudaStream_t s) {
  if (!x || !y) return fail(PMX_ERR_INVALID_ARGUMENT, "swiglu: null pointer");
  if (M <= 0 || D <= 0 || (D & 1)) return fail(PMX_ERR_INVALID_ARGUMENT, "swiglu: M>0 and an even D>0 required");
  PMX_DISPATCH_DTYPE(dtype, "swiglu", {
    const bool vec = (D / 2) % kVec<T> == 0 && aligned16(x) && aligned16(y);
    const int64_t items = M * (vec ? D / 2 / kVec<T> : D / 2);
    if (vec)
      PMX_PDL_LAUNCH((swiglu_kernel<T, true>), grid_for(items), kThreads, 0, s, (const T*)x, (T*)y, M, D, beta);
    else
      PMX_PDL_LAUNCH((swiglu_kernel<T, false>), grid_for(items), kThreads, 0, s, (const T*)x, (T*)y, M, D, beta);
  })
  return PMX_OK;
}

int launch_silu(const void* x, const void* gate, void* y, int64_t n, int dtype, cudaStream_t s) {
  if (!x || !y) return fail(PMX_ERR_INVALID_ARGUMENT, "silu: null pointer");
  if (n <= 0) return fail(PMX_ERR_INVALID_ARGUMENT, "silu: n must be positive");
  PMX_DISPATCH_DTYPE(dtype, "silu", {
    const bool vec = n % kVec<T> == 0 && aligned16(x) && aligned16(y) && (!gate || aligned16(gate));
    const int64_t items = vec ? n / kVec<T> : n;
    if (vec)
      PMX_PDL_LAUNCH((silu_kernel<T, true>), grid_for(items), kThreads, 0, s, (const T*)x, (const T*)gate, (T*)y, n);
    else
      PMX_PDL_LAUNCH((silu_kernel<T, false>), grid_for(items), kThreads, 0, s, (const T*)x, (const T*)gate, (T*)y, n);
  })
  return PMX_OK;
}

int launch_skip_rms_norm(const void* x, const void* skip, const void* weight, void* y, void* skip_out,
                         int64_t M, int64_t H, float eps, int dtype, cudaStream_t s) {
  if (!x || !weight || !y) return fail(PMX_ERR_INVALID_ARGUMENT, "skip_rms_norm: null pointer");
  if (skip && !skip_out) return fail(PMX_ERR_INVALID_ARGUMENT, "skip_rms_norm: skip_out is required when skip is given");
  if (M <= 0 || H <= 0) return fail(PMX_ERR_INVALID_ARGUMENT, "skip_rms_norm: M and H must be positive");
  int64_t blocks = M < (int64_t)sm_count() * 8 ? M : (int64_t)sm_count() * 8;
  PMX_DISPATCH_DTYPE(dtype, "skip_rms_norm", {
    const bool vec = H % kVec<T> == 0 && aligned16(x) && aligned16(y) && aligned16(weight) &&
                     (!skip || (aligned16(skip) && aligned16(skip_out)));
    T* so = skip ? (T*)skip_out : (T*)y;   // unused without skip
    if (vec && H / kVec<T> <= 32 * 16 && M >= 2048) {
      const int64_t wblocks = ceil_div(M, 8) < (int64_t)sm_count() * 8 ? ceil_div(M, 8) : (int64_t)sm_count() * 8;
      PMX_PDL_LAUNCH((skip_rms_norm_warp_kernel<T>), (int)wblocks, 256, 0, s, (const T*)x, (const T*)skip, (const T*)weight, (T*)y, so, M, H, eps);
    } else if (vec && H / kVec<T> <= 4 * 256)
      PMX_PDL_LAUNCH((skip_rms_norm_kernel<T, true, true>), (int)blocks, 256, 0, s, (const T*)x, (const T*)skip, (const T*)weight, (T*)y, so, M, H, eps);
    else if (vec)
      PMX_PDL_LAUNCH((skip_rms_norm_kernel<T, true, false>), (int)blocks, 256, 0, s, (const T*)x, (const T*)skip, (const T*)weight, (T*)y, so, M, H, eps);
    else
      PMX_PDL_LAUNCH((skip_rms_norm_kernel<T, false, false>), (int)blocks, 256, 0, s, (const T*)x, (const T*)skip, (const T*)weight, (T*)y, so, M, H, eps);
  })
  return PMX_OK;
}

int launch_zero_outside(void* y, const int64_t* off, int64_t M, int64_t n_out, int E, int dtype,
                        cudaStream_t s) {
  PMX_DISPATCH_DTYPE(dtype, "grouped_linear", {
    PMX_PDL_LAUNCH((zero_outside_kernel<T>), sm_count(), kThreads, 0, s, (T*)y, off, M, n_out, E);
  })
  return PMX_OK;
}

int launch_splitk_finish(const float* partial, const int64_t* off, const void* bias, void* y,
                         int64_t M, int64_t n_out, int E, int split, int dtype, bool swiglu,
                         float beta, cudaStream_t s) {
  if (n_out % 4) return fail(PMX_ERR_UNSUPPORTED, "grouped_linear: split-K needs N %% 4 == 0");
  PMX_DISPATCH_DTYPE(dtype, "grouped_linear", {
    if (swiglu)
      PMX_PDL_LAUNCH((splitk_finish_kernel<T, true>), grid_for(M * n_out / 4), kThreads, 0, s, partial, off, (const T*)bias, (T*)y, M, n_out, E, split, beta);
    else
      PMX_PDL_LAUNCH((splitk_finish_kernel<T, false>), grid_for(M * n_out / 4), kThreads, 0, s, partial, off, (const T*)bias, (T*)y, M, n_out, E, split, beta);
  })
  return PMX_OK;
}

}  // namespace pmx
