// moe_reduce fused with the tensor-parallel all-reduce, over NVLink peer memory.
//
// In the tensor-parallel MoE block every rank holds a partial down-projection
// y_r [T*k, N].  The result is  out[t] = sum_r sum_j w[t,j] * y_r[inv[t,j]]
// (MoeReduce.py:23-25 applied to the all-reduced rows of
// MoeRowParallelLinear.py:57-58; the weighted combine is linear, so it can run
// before the sum over ranks, which then moves [T,N] instead of [T*k,N]).
//
// One kernel per rank does both.  All ranks launch the same grid and walk the
// 16-byte items of the result in the same grid-stride order, so thread (b, i) of
// every rank owns the same items, and a CTA only ever waits for the same CTA of
// its peers: nothing depends on how many CTAs are resident on a GPU.
//
// Two exchange algorithms:
//
// PUSH (default): two hops, every word that crosses NVLink carries its own flag.
//   Items are dealt to owner ranks warp by warp (owner = (item / 32) % world).
//   1. every rank combines its partial of each item and stores it into the
//      owner's receive area A[source rank][slot] as 8-byte {data, epoch} words;
//   2. the owner polls the `world` slots of an item until all words show this
//      call's epoch, adds them in rank order (fp32), rounds once and stores the
//      result into receive area B[item] of every rank, again as {data, epoch};
//   3. every rank polls B for its items and writes `out`.
//   No fence and no separate flag: an 8-byte word is written atomically, so a
//   reader that sees the epoch sees the data.  Each rank sends and receives
//   2 x (world-1)/world x T*N*b x 2 bytes.
// PULL: one hop.  CTA b combines its slice into this rank's buffer, publishes an
//   epoch flag to every peer (st.release.sys), waits for CTA b of every peer and
//   sums the peers' buffers with 16-byte peer loads.  Each rank reads
//   (world-1) x T*N*b bytes.  Buffers alternate by epoch parity.
//
// Exchange buffer of a rank (the same layout on every rank; its size, not the
// current T, fixes the layout, so calls with different T can follow each other):
//   [0, 16384)            control: flags written by peers (PULL), epoch counter,
//                         exit ticket, status words, phase timestamps
//   [16384, 16384+R)      PUSH: receive area A      PULL: data buffer of even epochs
//   [16384+R, 16384+2R)   PUSH: receive area B      PULL: data buffer of odd epochs
// with R = ((buffer_bytes - 16384) / 2) rounded down to 256.
// Why a slot is never overwritten before it has been read (PUSH): a rank writes
// A slots of call n+1 only after it has finished call n, i.e. after it received
// every result of call n, each of which its owner produced after reading all A
// slots of that item; an owner writes B[item] of call n+1 on rank r only after
// it has r's partial of call n+1, which r sends after it finished call n.
//
// Waits are bounded (wait_limit_ns, default 1 s); on expiry the CTA records where
// it gave up in the status words and writes zeros to the items it still owed.
#include "common.cuh"

namespace pmx {
namespace {

constexpr int kMaxWorld = 8;   // one NVSwitch domain of B200s; also the unroll depth of the peer loads
constexpr int kMaxCtas = 320;  // grid limit: 2 CTAs on each of up to 160 SMs
constexpr size_t kCtrlBytes = 16384;
constexpr unsigned long long kDefaultWaitNs = 1000000000ull;

struct Ctrl {
  unsigned int epoch;             // last completed epoch of this rank
  unsigned int ticket_done;
  unsigned int pad0[62];
  int status[4];                  // code, peer, epoch, CTA
  unsigned int pad1[60];
  unsigned long long stamp[8];    // %globaltimer at the phase boundaries of CTA 0 (last call with stamps on)
  unsigned int pad2[48];
  unsigned int flags[kMaxWorld][kMaxCtas];  // PULL: flags[src][b] = last epoch CTA b of rank src published
};
static_assert(sizeof(Ctrl) <= kCtrlBytes, "control block too large");

struct Peers {
  char* base[kMaxWorld];
};

// Inputs and output of the rank(s) this launch plays.  A production launch plays
// one rank (gridDim.y == 1); the single-GPU emulation plays all ranks of the
// group in one cooperative launch, rank = blockIdx.y.
struct RankIO {
  const void* y[kMaxWorld];
  const void* w[kMaxWorld];
  const int64_t* inv[kMaxWorld];
  void* out[kMaxWorld];
  int rank0;
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
__device__ __forceinline__ void st_volatile16(void* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_volatile16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// 16 bytes of payload <-> one 32-byte slot of four {data, epoch} words
__device__ __forceinline__ void slot_store(char* slot, const uint4& d, unsigned int epoch) {
  st_volatile16(slot, make_uint4(d.x, epoch, d.y, epoch));
  st_volatile16(slot + 16, make_uint4(d.z, epoch, d.w, epoch));
}
__device__ __forceinline__ bool slot_ready(const uint4& a, const uint4& b, unsigned int epoch) {
  return a.y == epoch && a.w == epoch && b.y == epoch && b.w == epoch;
}

template <typename T>
__device__ __forceinline__ uint4 combine_item(const T* y, const T* w,
                                              const int64_t* inv, int k, int64_t N,
                                              int64_t t, int64_t c) {
  constexpr int V = kVec<T>;
  float acc[V];
#pragma unroll
  for (int v = 0; v < V; ++v) acc[v] = 0.f;
  for (int j = 0; j < k; ++j) {
    const int64_t r = inv[t * k + j];
    const float wj = Elem<T>::to_f(w[t * k + j]);
    float f[V];
    unpack16<T>(ld_stream16(y + r * N + c * V), f);
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = fmaf(wj, f[v], acc[v]);
  }
  return pack16<T>(acc);
}

__device__ __forceinline__ void record_timeout(Ctrl* ctrl, int peer, unsigned int epoch) {
  if (atomicCAS(&ctrl->status[0], 0, 1) == 0) {
    ctrl->status[1] = peer;
    ctrl->status[2] = (int)epoch;
    ctrl->status[3] = blockIdx.x;
  }
}

// epoch of this call (every CTA reads the counter the last CTA of the previous
// call advanced) and the abort flag
__device__ __forceinline__ unsigned int begin_call(Ctrl* ctrl, unsigned int* s_epoch, volatile int* s_abort) {
  if (threadIdx.x == 0) {
    *s_epoch = *reinterpret_cast<volatile unsigned int*>(&ctrl->epoch) + 1u;
    *s_abort = 0;
  }
  __syncthreads();
  return *s_epoch;
}
__device__ __forceinline__ void end_call(Ctrl* ctrl, unsigned int epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(&ctrl->ticket_done, 1u);
    if (done == gridDim.x - 1) {
      ctrl->ticket_done = 0;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(&ctrl->epoch) = epoch;
    }
  }
}

// ----------------------------------------------------------------------------- PUSH
template <typename T, bool STAMPS>
__global__ void __launch_bounds__(256, 2)
combine_allreduce_push_kernel(RankIO io, int64_t Tn, int k, int64_t N, Peers peers, int world,
                              size_t region, unsigned long long wait_ns) {
  constexpr int V = kVec<T>;
  __shared__ unsigned int s_epoch;
  __shared__ volatile int s_abort;
  pdl_launch_dependents();
  pdl_wait();   // y, w and inv come from the kernels in front of this one
  const int rank = io.rank0 + blockIdx.y;
  const T* y = reinterpret_cast<const T*>(io.y[blockIdx.y]);
  const T* w = reinterpret_cast<const T*>(io.w[blockIdx.y]);
  const int64_t* inv = io.inv[blockIdx.y];
  T* out = reinterpret_cast<T*>(io.out[blockIdx.y]);
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(peers.base[rank]);
  const unsigned int epoch = begin_call(ctrl, &s_epoch, &s_abort);
  const bool stamper = STAMPS && blockIdx.x == 0 && threadIdx.x == 0;
  if (stamper) ctrl->stamp[0] = now_ns();

  const int64_t chunks = N / V, total = Tn * chunks;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;   // a multiple of 32: item / 32 is the same for a warp
  const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  // slots per source rank in receive area A: what the largest T that fits this buffer needs
  const int64_t own_slots = (int64_t)(region / 32 / world) & ~int64_t(31);

  // 1. combine my partial of every item and hand it to the item's owner
  for (int64_t i = first; i < total; i += stride) {
    const int64_t t = i / chunks, c = i - t * chunks;
    const uint4 mine = combine_item<T>(y, w, inv, k, N, t, c);
    const int64_t g = i >> 5;
    const int owner = (int)(g % world);
    const int64_t j = (g / world) * 32 + (i & 31);
    slot_store(peers.base[owner] + kCtrlBytes + ((size_t)rank * own_slots + j) * 32, mine, epoch);
  }
  if (stamper) ctrl->stamp[1] = now_ns();

  // 2. owner: collect the partials of all ranks, add, publish the sum to every rank
  for (int64_t i = first; i < total; i += stride) {
    const int64_t g = i >> 5;
    if ((int)(g % world) != rank) continue;
    const int64_t j = (g / world) * 32 + (i & 31);
    const char* slots = peers.base[rank] + kCtrlBytes + (size_t)j * 32;
    uint4 a[kMaxWorld], b[kMaxWorld];
    unsigned int pending = (1u << world) - 1u;
    const unsigned long long t0 = now_ns();
    unsigned int it = 0;
    while (true) {
#pragma unroll
      for (int p = 0; p < kMaxWorld; ++p) {
        if (p < world && ((pending >> p) & 1u)) {
          const char* s = slots + (size_t)p * own_slots * 32;
          a[p] = ld_volatile16(s);
          b[p] = ld_volatile16(s + 16);
        }
      }
#pragma unroll
      for (int p = 0; p < kMaxWorld; ++p)
        if (p < world && ((pending >> p) & 1u) && slot_ready(a[p], b[p], epoch)) pending &= ~(1u << p);
      if (!pending) break;
      if ((++it & 127u) == 0u && (s_abort || now_ns() - t0 > wait_ns)) {
        s_abort = 1;
        record_timeout(ctrl, __ffs(pending) - 1, epoch);
        break;
      }
    }
    float acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = 0.f;
    if (!pending) {
#pragma unroll
      for (int p = 0; p < kMaxWorld; ++p) {
        if (p < world) {
          float f[V];
          unpack16<T>(make_uint4(a[p].x, a[p].z, b[p].x, b[p].z), f);
#pragma unroll
          for (int v = 0; v < V; ++v) acc[v] += f[v];
        }
      }
    }
    const uint4 sum = pack16<T>(acc);   // zeros after a timeout
    reinterpret_cast<uint4*>(out)[i] = sum;
    if (!pending) {
#pragma unroll
      for (int p = 0; p < kMaxWorld; ++p)
        if (p < world && p != rank) slot_store(peers.base[p] + kCtrlBytes + region + (size_t)i * 32, sum, epoch);
    }
  }
  if (stamper) ctrl->stamp[2] = now_ns();

  // 3. everybody: pick up the sums of the items other ranks own
  for (int64_t i = first; i < total; i += stride) {
    const int64_t g = i >> 5;
    if ((int)(g % world) == rank) continue;
    const char* slot = peers.base[rank] + kCtrlBytes + region + (size_t)i * 32;
    uint4 a, b;
    const unsigned long long t0 = now_ns();
    unsigned int it = 0;
    bool ok = true;
    while (true) {
      a = ld_volatile16(slot);
      b = ld_volatile16(slot + 16);
      if (slot_ready(a, b, epoch)) break;
      if ((++it & 127u) == 0u && (s_abort || now_ns() - t0 > wait_ns)) {
        s_abort = 1;
        record_timeout(ctrl, (int)(g % world), epoch);
        ok = false;
        break;
      }
    }
    reinterpret_cast<uint4*>(out)[i] = ok ? make_uint4(a.x, a.z, b.x, b.z) : make_uint4(0, 0, 0, 0);
  }
  if (stamper) {
    ctrl->stamp[3] = now_ns();
    ctrl->stamp[4] = ctrl->stamp[3];
  }
  end_call(ctrl, epoch);
}

// ----------------------------------------------------------------------------- PULL
template <typename T, bool STAMPS>
__global__ void __launch_bounds__(256, 2)
combine_allreduce_pull_kernel(RankIO io, int64_t Tn, int k, int64_t N, Peers peers, int world,
                              size_t region, unsigned long long wait_ns) {
  constexpr int V = kVec<T>;
  __shared__ unsigned int s_epoch;
  __shared__ volatile int s_abort;
  pdl_launch_dependents();
  pdl_wait();
  const int rank = io.rank0 + blockIdx.y;
  const T* y = reinterpret_cast<const T*>(io.y[blockIdx.y]);
  const T* w = reinterpret_cast<const T*>(io.w[blockIdx.y]);
  const int64_t* inv = io.inv[blockIdx.y];
  T* out = reinterpret_cast<T*>(io.out[blockIdx.y]);
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(peers.base[rank]);
  const unsigned int epoch = begin_call(ctrl, &s_epoch, &s_abort);
  const bool stamper = STAMPS && blockIdx.x == 0 && threadIdx.x == 0;
  if (stamper) ctrl->stamp[0] = now_ns();
  const size_t data_off = kCtrlBytes + (epoch & 1u) * region;
  const int64_t chunks = N / V, total = Tn * chunks;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;

  // 1. local weighted combine -> my exchange buffer
  uint4* mine = reinterpret_cast<uint4*>(peers.base[rank] + data_off);
  for (int64_t i = first; i < total; i += stride) {
    const int64_t t = i / chunks, c = i - t * chunks;
    mine[i] = combine_item<T>(y, w, inv, k, N, t, c);
  }
  __syncthreads();   // the block's stores to the exchange buffer are done (CTA scope)
  if (stamper) ctrl->stamp[1] = now_ns();
  // 2. publish: my slice of this rank's buffer is complete (thread p tells peer p).  The
  // release store orders the whole block's buffer stores before the flag: they
  // happen-before this thread through the barrier above.
  if (threadIdx.x < world && threadIdx.x != rank)
    st_release_sys(&reinterpret_cast<Ctrl*>(peers.base[threadIdx.x])->flags[rank][blockIdx.x], epoch);
  if (stamper) ctrl->stamp[2] = now_ns();
  // 3. wait until the same CTA of every peer has published this epoch
  if (threadIdx.x < world && threadIdx.x != rank) {
    const unsigned int* flag = &ctrl->flags[threadIdx.x][blockIdx.x];
    const unsigned long long t0 = now_ns();
    unsigned int it = 0;
    while ((int)(ld_acquire_sys(flag) - epoch) < 0) {
      if ((++it & 255u) == 0u && now_ns() - t0 > wait_ns) {
        s_abort = 1;
        record_timeout(ctrl, threadIdx.x, epoch);
        break;
      }
    }
  }
  __syncthreads();
  if (stamper) ctrl->stamp[3] = now_ns();
  // 4. sum over ranks (zeros when a peer never arrived)
  const bool aborted = s_abort != 0;
  for (int64_t i = first; i < total; i += stride) {
    // issue the loads from all ranks before using any of them: NVLink latency
    // is paid once per item, not once per rank
    uint4 raw[kMaxWorld];
    float acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = 0.f;
    if (!aborted) {
#pragma unroll
      for (int p = 0; p < kMaxWorld; ++p)
        if (p < world) raw[p] = __ldcg(reinterpret_cast<const uint4*>(peers.base[p] + data_off) + i);
#pragma unroll
      for (int p = 0; p < kMaxWorld; ++p) {
        if (p < world) {
          float f[V];
          unpack16<T>(raw[p], f);
#pragma unroll
          for (int v = 0; v < V; ++v) acc[v] += f[v];
        }
      }
    }
    reinterpret_cast<uint4*>(out)[i] = pack16<T>(acc);
  }
  if (stamper) ctrl->stamp[4] = now_ns();
  end_call(ctrl, epoch);
}

size_t region_of(size_t buffer_bytes) {
  return buffer_bytes > kCtrlBytes ? (((buffer_bytes - kCtrlBytes) / 2) & ~size_t(255)) : 0;
}

template <typename T>
int launch_typed(const RankIO& io, int nranks_here, int64_t Tn, int k, int64_t N, const Peers& peers, int world,
                 size_t region, int algo, bool stamps, unsigned long long wait_ns, int blocks, cudaStream_t s) {
  const void* kern;
  if (algo == PMX_ALLREDUCE_PULL)
    kern = stamps ? (const void*)combine_allreduce_pull_kernel<T, true> : (const void*)combine_allreduce_pull_kernel<T, false>;
  else
    kern = stamps ? (const void*)combine_allreduce_push_kernel<T, true> : (const void*)combine_allreduce_push_kernel<T, false>;
  void* args[] = {(void*)&io, (void*)&Tn, (void*)&k, (void*)&N, (void*)&peers, (void*)&world, (void*)&region, (void*)&wait_ns};
  if (nranks_here > 1) {
    // all ranks of the group in one launch on one GPU: their CTAs wait for one
    // another, so they must be resident together
    PMX_CUDA_OK(cudaLaunchCooperativeKernel(kern, dim3(blocks, nranks_here), dim3(256), args, 0, s));
    count_launches(1);
    return PMX_OK;
  }
  return launch_pdl(kern, dim3(blocks), dim3(256), 0, s, args);
}

int check_common(int64_t Tn, int k, int64_t N, int dtype, void* const* peer_buffers, int world, size_t buffer_bytes,
                 int algo, Peers* peers, size_t* region) {
  if (!peer_buffers) return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce_allreduce: null pointer");
  if (Tn <= 0 || k <= 0 || N <= 0) return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce_allreduce: T, k, N must be positive");
  if (world < 1 || world > kMaxWorld)
    return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce_allreduce: world %d out of range (at most %d ranks)", world, kMaxWorld);
  if (algo != PMX_ALLREDUCE_AUTO && algo != PMX_ALLREDUCE_PULL && algo != PMX_ALLREDUCE_PUSH)
    return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce_allreduce: unknown algorithm %d", algo);
  const size_t need = reduce_allreduce_buffer_bytes(Tn, N, dtype);
  if (buffer_bytes < need)
    return fail(PMX_ERR_WORKSPACE, "moe_reduce_allreduce: exchange buffers of %zu bytes needed, %zu given", need, buffer_bytes);
  const int vec = dtype == PMX_DTYPE_F32 ? 4 : 8;
  if (N % vec) return fail(PMX_ERR_ALIGNMENT, "moe_reduce_allreduce: N must be a multiple of %d elements", vec);
  for (int p = 0; p < world; ++p) {
    if (!peer_buffers[p] || !aligned16(peer_buffers[p]))
      return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce_allreduce: exchange buffer of rank %d missing or misaligned", p);
    peers->base[p] = reinterpret_cast<char*>(peer_buffers[p]);
  }
  *region = region_of(buffer_bytes);
  return PMX_OK;
}

int grid_blocks(int64_t Tn, int64_t N, int dtype) {
  const int vec = dtype == PMX_DTYPE_F32 ? 4 : 8;
  const int64_t items = Tn * (N / vec);
  int64_t blocks = ceil_div(items, 256);
  // the same grid on every rank (it depends only on T, N and the SM count): thread
  // (b, i) of each rank owns the same items
  if (blocks > 2 * (int64_t)sm_count()) blocks = 2 * (int64_t)sm_count();
  if (blocks > kMaxCtas) blocks = kMaxCtas;
  return (int)blocks;
}

int dispatch(const RankIO& io, int nranks_here, int64_t Tn, int k, int64_t N, int dtype, const Peers& peers, int world,
             size_t region, int algo, int flags, long long wait_limit_ns, int blocks, cudaStream_t s) {
  if (algo == PMX_ALLREDUCE_AUTO) algo = PMX_ALLREDUCE_PUSH;
  const bool stamps = (flags & PMX_ALLREDUCE_FLAG_STAMPS) != 0;
  const unsigned long long wait_ns = wait_limit_ns > 0 ? (unsigned long long)wait_limit_ns : kDefaultWaitNs;
  switch (dtype) {
    case PMX_DTYPE_F16: return launch_typed<__half>(io, nranks_here, Tn, k, N, peers, world, region, algo, stamps, wait_ns, blocks, s);
    case PMX_DTYPE_BF16: return launch_typed<__nv_bfloat16>(io, nranks_here, Tn, k, N, peers, world, region, algo, stamps, wait_ns, blocks, s);
    case PMX_DTYPE_F32: return launch_typed<float>(io, nranks_here, Tn, k, N, peers, world, region, algo, stamps, wait_ns, blocks, s);
  }
  return fail(PMX_ERR_UNSUPPORTED, "moe_reduce_allreduce: unknown dtype %d", dtype);
}

}  // namespace

size_t reduce_allreduce_buffer_bytes(int64_t T, int64_t N, int dtype) {
  const int vec = dtype == PMX_DTYPE_F32 ? 4 : 8;
  const size_t items = (size_t)ceil_div(T * N, vec);
  // one 32-byte slot per item in each of the two areas, plus the rounding of the
  // per-rank slices of area A to whole warps
  const size_t region = (size_t)ceil_div((int64_t)((items + 32 * kMaxWorld) * 32), 256) * 256;
  return kCtrlBytes + 2 * region;
}

int launch_reduce_allreduce(const void* y, const void* w, const int64_t* inv, void* out, int64_t Tn,
                            int k, int64_t N, int dtype, void* const* peer_buffers, int rank,
                            int world, size_t buffer_bytes, int algo, int flags, long long wait_limit_ns,
                            cudaStream_t s) {
  if (!y || !w || !inv || !out) return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce_allreduce: null pointer");
  Peers peers{};
  size_t region = 0;
  const int st = check_common(Tn, k, N, dtype, peer_buffers, world, buffer_bytes, algo, &peers, &region);
  if (st != PMX_OK) return st;
  if (rank < 0 || rank >= world)
    return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce_allreduce: rank %d out of range for %d ranks", rank, world);
  if (!aligned16(y) || !aligned16(out))
    return fail(PMX_ERR_ALIGNMENT, "moe_reduce_allreduce: y and out must be 16-byte aligned");
  RankIO io{};
  io.y[0] = y; io.w[0] = w; io.inv[0] = inv; io.out[0] = out; io.rank0 = rank;
  return dispatch(io, 1, Tn, k, N, dtype, peers, world, region, algo, flags, wait_limit_ns, grid_blocks(Tn, N, dtype), s);
}

int launch_reduce_allreduce_emulated(const void* const* y, const void* const* w, const int64_t* const* inv,
                                     void* const* out, int64_t Tn, int k, int64_t N, int dtype,
                                     void* const* buffers, int world, size_t buffer_bytes, int algo,
                                     long long wait_limit_ns, cudaStream_t s) {
  if (!y || !w || !inv || !out) return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce_allreduce_emulated: null pointer");
  Peers peers{};
  size_t region = 0;
  const int st = check_common(Tn, k, N, dtype, buffers, world, buffer_bytes, algo, &peers, &region);
  if (st != PMX_OK) return st;
  RankIO io{};
  for (int r = 0; r < world; ++r) {
    if (!y[r] || !w[r] || !inv[r] || !out[r] || !aligned16(y[r]) || !aligned16(out[r]))
      return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce_allreduce_emulated: tensors of rank %d missing or misaligned", r);
    io.y[r] = y[r]; io.w[r] = w[r]; io.inv[r] = inv[r]; io.out[r] = out[r];
  }
  io.rank0 = 0;
  // every CTA of every emulated rank must be resident at once: cap the grid
  int blocks = grid_blocks(Tn, N, dtype);
  const int cap = 2 * sm_count() / world;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return dispatch(io, world, Tn, k, N, dtype, peers, world, region, algo, 0, wait_limit_ns, blocks, s);
}

int reduce_allreduce_check(void* my_buffer, int out[4], cudaStream_t s) {
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(my_buffer);
  PMX_CUDA_OK(cudaMemcpyAsync(out, ctrl->status, 4 * sizeof(int), cudaMemcpyDeviceToHost, s));
  PMX_CUDA_OK(cudaStreamSynchronize(s));
  if (out[0] != 0) {
    // reported once: clear the record so that later calls are judged on their own
    PMX_CUDA_OK(cudaMemsetAsync(ctrl->status, 0, 4 * sizeof(int), s));
    PMX_CUDA_OK(cudaStreamSynchronize(s));
    return fail(PMX_ERR_DEVICE_CHECK, "moe_reduce_allreduce: gave up waiting for rank %d in epoch %d (CTA %d)", out[1], out[2], out[3]);
  }
  return PMX_OK;
}

int reduce_allreduce_phases(const void* my_buffer, unsigned long long out[8], cudaStream_t s) {
  const Ctrl* ctrl = reinterpret_cast<const Ctrl*>(my_buffer);
  PMX_CUDA_OK(cudaMemcpyAsync(out, ctrl->stamp, 8 * sizeof(unsigned long long), cudaMemcpyDeviceToHost, s));
  PMX_CUDA_OK(cudaStreamSynchronize(s));
  return PMX_OK;
}

}  // namespace pmx
