// CUDA-core grouped expert GEMM with exact fp32 multiply-accumulate.
//
// This is the kernel for float32 tensors (the tensor-core path would have to
// round fp32 operands to tf32) and for shapes the tcgen05 kernel does not take
// (K or N not a multiple of 8 elements).  Same contract as the tensor-core
// kernel: y[r,:] = x[r,:] . w[e]^T (+ bias[e]) for rows r of expert e, optional
// fused SwiGLU, offsets read on the device.
#include "common.cuh"

namespace pmx {
namespace {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename T, bool SWIGLU>
__global__ void __launch_bounds__(256)
grouped_gemm_simt_kernel(const T* __restrict__ x, const int64_t* __restrict__ off,
                         const T* __restrict__ w, const T* __restrict__ bias, T* __restrict__ y,
                         int64_t M, int N, int K, int E, float beta, int64_t w_pitch) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  __shared__ float Bu[SWIGLU ? BK : 1][BN + 4];
  __shared__ int s_expert, s_row0, s_row_end;

  const int n_out = SWIGLU ? N / 2 : N;
  // which (expert, row tile) does blockIdx.y stand for?
  if (threadIdx.x == 0) {
    int64_t tile = blockIdx.y;
    int e = 0;
    s_expert = -1;
    for (; e < E; ++e) {
      int64_t r0 = offset_at(off, e, M), r1 = offset_at(off, e + 1, M);
      r0 = r0 < 0 ? 0 : r0;
      r1 = r1 > M ? M : r1;
      const int64_t tiles = r1 > r0 ? (r1 - r0 + BM - 1) / BM : 0;
      if (tile < tiles) {
        s_expert = e;
        s_row0 = (int)(r0 + tile * BM);
        s_row_end = (int)r1;
        break;
      }
      tile -= tiles;
    }
  }
  __syncthreads();
  const int e = s_expert;
  if (e < 0) return;
  const int row0 = s_row0, row_end = s_row_end;
  const int n0 = blockIdx.x * BN;
  const T* we = w + (int64_t)e * w_pitch * K;

  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4] = {}, accu[4][4] = {};
  const int lr = threadIdx.x / 4;        // 0..63: tile row loaded by this thread
  const int lk = (threadIdx.x % 4) * 4;  // 0,4,8,12: first k of its 4 elements

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int kk = k0 + lk + i;
      const int r = row0 + lr;
      As[lk + i][lr] = (r < row_end && kk < K) ? Elem<T>::to_f(x[(int64_t)r * K + kk]) : 0.f;
      const int n = n0 + lr;
      Bs[lk + i][lr] = (n < n_out && kk < K) ? Elem<T>::to_f(we[(int64_t)n * K + kk]) : 0.f;
      if (SWIGLU)
        Bu[lk + i][lr] = (n < n_out && kk < K) ? Elem<T>::to_f(we[(int64_t)(n_out + n) * K + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4], u[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = As[kk][ty * 4 + i];
        b[i] = Bs[kk][tx * 4 + i];
        if (SWIGLU) u[i] = Bu[kk][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (SWIGLU) accu[i][j] = fmaf(a[i], u[j], accu[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + ty * 4 + i;
    if (r >= row_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= n_out) continue;
      float v = acc[i][j];
      if (bias) v += Elem<T>::to_f(bias[(int64_t)e * w_pitch + n]);
      if (SWIGLU) {
        float u = accu[i][j];
        if (bias) u += Elem<T>::to_f(bias[(int64_t)e * w_pitch + n_out + n]);
        v = u * v / (1.0f + expf(-beta * v));
      }
      y[(int64_t)r * n_out + n] = Elem<T>::from_f(v);
    }
  }
}

template <typename T>
int run(const void* x, const int64_t* off, const void* w, const void* bias, void* y, int64_t M,
        int64_t N, int64_t K, int E, int epilogue, float beta, int64_t w_pitch, cudaStream_t s) {
  const int64_t n_out = epilogue == PMX_EPILOGUE_SWIGLU ? N / 2 : N;
  const int64_t row_tiles = ceil_div(M, BM) + E;  // upper bound on ragged row tiles
  if (row_tiles > 65535) return fail(PMX_ERR_UNSUPPORTED, "grouped_linear (CUDA-core kernel): too many rows (%lld)", (long long)M);
  dim3 grid((unsigned)ceil_div(n_out, BN), (unsigned)row_tiles);
  if (epilogue == PMX_EPILOGUE_SWIGLU)
    grouped_gemm_simt_kernel<T, true><<<grid, 256, 0, s>>>((const T*)x, off, (const T*)w, (const T*)bias, (T*)y, M, (int)N, (int)K, E, beta, w_pitch);
  else
    grouped_gemm_simt_kernel<T, false><<<grid, 256, 0, s>>>((const T*)x, off, (const T*)w, (const T*)bias, (T*)y, M, (int)N, (int)K, E, beta, w_pitch);
  PMX_LAUNCHED();
  return PMX_OK;
}

}  // namespace

int launch_gemm_simt(const void* x, const int64_t* off, const void* w, const void* bias, void* y,
                     int64_t M, int64_t N, int64_t K, int E, int dtype, int epilogue, float beta,
                     int64_t w_pitch, cudaStream_t s) {
  if (w_pitch <= 0) w_pitch = N;
  switch (dtype) {
    case PMX_DTYPE_F16: return run<__half>(x, off, w, bias, y, M, N, K, E, epilogue, beta, w_pitch, s);
    case PMX_DTYPE_BF16: return run<__nv_bfloat16>(x, off, w, bias, y, M, N, K, E, epilogue, beta, w_pitch, s);
    case PMX_DTYPE_F32: return run<float>(x, off, w, bias, y, M, N, K, E, epilogue, beta, w_pitch, s);
  }
  return fail(PMX_ERR_UNSUPPORTED, "grouped_linear: unknown dtype %d", dtype);
}

}  // namespace pmx
