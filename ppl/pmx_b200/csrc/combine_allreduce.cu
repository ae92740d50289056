// moe_reduce fused with the tensor-parallel all-reduce, over NVLink peer memory.
//
// In the tensor-parallel MoE block every rank holds a partial down-projection
// y_r [T*k, N].  The result is  out[t] = sum_r sum_j w[t,j] * y_r[inv[t,j]]
// (MoeReduce.py:23-25 applied to the all-reduced rows of
// MoeRowParallelLinear.py:57-58; the weighted combine is linear, so it can run
// before the sum over ranks, which then moves [T,N] instead of [T*k,N]).
//
// One kernel per rank does both, CTA by CTA.  All ranks launch the same grid and
// walk the rows in the same grid-stride order, so CTA b of every rank owns the
// same slice of the result:
//   1. CTA b combines its slice of the local rows into this rank's exchange
//      buffer (T1, fp32 math);
//   2. it publishes the epoch number in flag [rank][b] of every peer (release,
//      system scope);
//   3. it waits (bounded) until flag [p][b] of its own control block shows this
//      epoch for every peer p, i.e. until CTA b of every peer has done step 1;
//   4. it sums its slice over all ranks' buffers, reading the peers' buffers
//      with plain 16-byte loads over NVLink, and writes `out`.
// No CTA waits for another CTA of its own GPU, so nothing depends on how many
// CTAs are resident.  One-shot exchange: each rank pulls (world-1) * T*N*b
// bytes, which is the right trade below a few MB (decode); larger messages stay
// with NCCL.
//
// Exchange buffer of a rank (the same layout on every rank, allocated
// symmetrically by the host side):
//   [0, 16384)     control: flags[src rank][CTA] written by peers, epoch counter,
//                  exit ticket, status words, phase timestamps
//   [16384, ...)   two data buffers used alternately (epoch parity), so a rank
//                  may start the next call while a slower peer still reads the
//                  previous one.
// Waits are bounded to 1 s; on expiry the CTA records where it gave up in the
// status words and skips its sum.
#include "common.cuh"

namespace pmx {
namespace {

constexpr int kMaxWorld = 8;   // one NVSwitch domain of B200s; also the unroll depth of the peer loads
constexpr int kMaxCtas = 320;  // grid limit: 2 CTAs on each of up to 160 SMs
constexpr size_t kCtrlBytes = 16384;
constexpr unsigned long long kWaitNs = 1000000000ull;

struct Ctrl {
  unsigned int epoch;             // last completed epoch of this rank
  unsigned int ticket_done;
  unsigned int pad0[62];
  int status[4];                  // code, peer, epoch, CTA
  unsigned int pad1[60];
  unsigned long long stamp[8];    // %globaltimer at the phase boundaries of CTA 0 (last call)
  unsigned int pad2[48];
  unsigned int flags[kMaxWorld][kMaxCtas];  // flags[src][b] = last epoch CTA b of rank src published
};
static_assert(sizeof(Ctrl) <= kCtrlBytes, "control block too large");

struct Peers {
  char* base[kMaxWorld];
};

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <typename T>
__global__ void __launch_bounds__(256, 2)
combine_allreduce_kernel(const T* __restrict__ y, const T* __restrict__ w,
                         const int64_t* __restrict__ inv, T* __restrict__ out, int64_t Tn, int k,
                         int64_t N, Peers peers, int rank, int world, size_t data_bytes) {
  constexpr int V = kVec<T>;
  __shared__ unsigned int s_epoch;
  __shared__ int s_abort;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(peers.base[rank]);
  if (threadIdx.x == 0) {
    s_epoch = *reinterpret_cast<volatile unsigned int*>(&ctrl->epoch) + 1u;
    s_abort = 0;
  }
  __syncthreads();
  const bool stamper = blockIdx.x == 0 && threadIdx.x == 0;
  if (stamper) ctrl->stamp[0] = now_ns();
  const unsigned int epoch = s_epoch;
  const size_t data_off = kCtrlBytes + (epoch & 1u) * data_bytes;
  const int64_t chunks = N / V, total = Tn * chunks;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;

  // 1. local weighted combine -> my exchange buffer
  T* mine = reinterpret_cast<T*>(peers.base[rank] + data_off);
  for (int64_t i = first; i < total; i += stride) {
    const int64_t t = i / chunks, c = i - t * chunks;
    float acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = 0.f;
    for (int j = 0; j < k; ++j) {
      const int64_t r = inv[t * k + j];
      const float wj = Elem<T>::to_f(w[t * k + j]);
      float f[V];
      unpack16<T>(ld_nc16(y + r * N + c * V), f);
#pragma unroll
      for (int v = 0; v < V; ++v) acc[v] = fmaf(wj, f[v], acc[v]);
    }
    *reinterpret_cast<uint4*>(mine + t * N + c * V) = pack16<T>(acc);
  }
  __syncthreads();   // the block's stores to the exchange buffer are done (CTA scope)
  if (stamper) ctrl->stamp[1] = now_ns();
  // 2. publish: my slice of this rank's buffer is complete (thread p tells peer p)
  // (the release store orders the whole block's buffer stores before the flag: they
  // happen-before this thread through the barrier above)
  if (threadIdx.x < world && threadIdx.x != rank) {
    st_release_sys(&reinterpret_cast<Ctrl*>(peers.base[threadIdx.x])->flags[rank][blockIdx.x], epoch);
  }
  if (stamper) ctrl->stamp[2] = now_ns();
  // 3. wait until the same CTA of every peer has published this epoch
  if (threadIdx.x < world && threadIdx.x != rank) {
    const unsigned int* flag = &ctrl->flags[threadIdx.x][blockIdx.x];
    const unsigned long long t0 = now_ns();
    unsigned int it = 0;
    while ((int)(ld_acquire_sys(flag) - epoch) < 0) {
      if ((++it & 255u) == 0u && now_ns() - t0 > kWaitNs) {
        s_abort = 1;
        if (atomicCAS(&ctrl->status[0], 0, 1) == 0) {
          ctrl->status[1] = threadIdx.x;
          ctrl->status[2] = (int)epoch;
          ctrl->status[3] = blockIdx.x;
        }
        break;
      }
    }
  }
  __syncthreads();
  if (stamper) ctrl->stamp[3] = now_ns();
  // 4. sum over ranks
  if (!s_abort) {
    for (int64_t i = first; i < total; i += stride) {
      // issue the loads from all ranks before using any of them: NVLink latency
      // is paid once per item, not once per rank
      uint4 raw[kMaxWorld];
#pragma unroll
      for (int p = 0; p < kMaxWorld; ++p)
        if (p < world) raw[p] = __ldcg(reinterpret_cast<const uint4*>(peers.base[p] + data_off) + i);
      float acc[V];
#pragma unroll
      for (int v = 0; v < V; ++v) acc[v] = 0.f;
#pragma unroll
      for (int p = 0; p < kMaxWorld; ++p) {
        if (p < world) {
          float f[V];
          unpack16<T>(raw[p], f);
#pragma unroll
          for (int v = 0; v < V; ++v) acc[v] += f[v];
        }
      }
      reinterpret_cast<uint4*>(out)[i] = pack16<T>(acc);
    }
  }
  __syncthreads();
  if (stamper) ctrl->stamp[4] = now_ns();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(&ctrl->ticket_done, 1u);
    if (done == gridDim.x - 1) {
      ctrl->ticket_done = 0;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(&ctrl->epoch) = epoch;
    }
  }
}

}  // namespace

size_t reduce_allreduce_buffer_bytes(int64_t T, int64_t N, int dtype) {
  const size_t b = dtype == PMX_DTYPE_F32 ? 4 : 2;
  const size_t data = (size_t)ceil_div((int64_t)(T * N * b), 256) * 256;
  return kCtrlBytes + 2 * data;
}

int launch_reduce_allreduce(const void* y, const void* w, const int64_t* inv, void* out, int64_t Tn,
                            int k, int64_t N, int dtype, void* const* peer_buffers, int rank,
                            int world, size_t buffer_bytes, cudaStream_t s) {
  if (!y || !w || !inv || !out || !peer_buffers)
    return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce_allreduce: null pointer");
  if (Tn <= 0 || k <= 0 || N <= 0) return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce_allreduce: T, k, N must be positive");
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world)
    return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce_allreduce: rank %d / world %d out of range (at most %d ranks)", rank, world, kMaxWorld);
  const size_t need = reduce_allreduce_buffer_bytes(Tn, N, dtype);
  if (buffer_bytes < need)
    return fail(PMX_ERR_WORKSPACE, "moe_reduce_allreduce: exchange buffers of %zu bytes needed, %zu given", need, buffer_bytes);
  const int vec = dtype == PMX_DTYPE_F32 ? 4 : 8;
  if (N % vec || !aligned16(y) || !aligned16(out))
    return fail(PMX_ERR_ALIGNMENT, "moe_reduce_allreduce: N must be a multiple of %d elements and y, out 16-byte aligned", vec);
  Peers peers{};
  for (int p = 0; p < world; ++p) {
    if (!peer_buffers[p] || !aligned16(peer_buffers[p]))
      return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce_allreduce: exchange buffer of rank %d missing or misaligned", p);
    peers.base[p] = reinterpret_cast<char*>(peer_buffers[p]);
  }
  const size_t data_bytes = (need - kCtrlBytes) / 2;
  const int64_t items = Tn * (N / vec);
  int64_t blocks = ceil_div(items, 256);
  // the same grid on every rank (it depends only on T, N and the SM count): CTA b of
  // each rank owns the same rows
  if (blocks > 2 * (int64_t)sm_count()) blocks = 2 * (int64_t)sm_count();
  if (blocks > kMaxCtas) blocks = kMaxCtas;
  switch (dtype) {
    case PMX_DTYPE_F16:
      combine_allreduce_kernel<__half><<<(int)blocks, 256, 0, s>>>((const __half*)y, (const __half*)w, inv, (__half*)out, Tn, k, N, peers, rank, world, data_bytes);
      break;
    case PMX_DTYPE_BF16:
      combine_allreduce_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, s>>>((const __nv_bfloat16*)y, (const __nv_bfloat16*)w, inv, (__nv_bfloat16*)out, Tn, k, N, peers, rank, world, data_bytes);
      break;
    case PMX_DTYPE_F32:
      combine_allreduce_kernel<float><<<(int)blocks, 256, 0, s>>>((const float*)y, (const float*)w, inv, (float*)out, Tn, k, N, peers, rank, world, data_bytes);
      break;
    default:
      return fail(PMX_ERR_UNSUPPORTED, "moe_reduce_allreduce: unknown dtype %d", dtype);
  }
  PMX_LAUNCHED();
  return PMX_OK;
}

int reduce_allreduce_check(const void* my_buffer, int out[4], cudaStream_t s) {
  const Ctrl* ctrl = reinterpret_cast<const Ctrl*>(my_buffer);
  PMX_CUDA_OK(cudaMemcpyAsync(out, ctrl->status, 4 * sizeof(int), cudaMemcpyDeviceToHost, s));
  PMX_CUDA_OK(cudaStreamSynchronize(s));
  if (out[0] != 0)
    return fail(PMX_ERR_DEVICE_CHECK, "moe_reduce_allreduce: gave up waiting for rank %d in epoch %d (CTA %d)", out[1], out[2], out[3]);
  return PMX_OK;
}

}  // namespace pmx
