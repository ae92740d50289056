// moe_select on the GPU: router top-k + softmax, per-expert histogram, prefix
// offsets, stable permutation and the 128-bit vectorised token gather.
//
// Replaces MoeSelect.forward (torch_function/MoeSelect.py:36-64).  No host
// synchronisation and no order-dependent atomics anywhere: the permutation is a
// pure function of the scores, so every tensor-parallel rank computes the same
// routing bit for bit.  Three code paths share the ranking rule (higher score
// first, lower expert index among equals):
//
// Large batches, three launches:
//   route_count : one warp per token picks the k best experts, writes the
//                 softmax of the k kept logits and the expert ids; each block of
//                 `tpb` tokens leaves its per-expert row count.
//   scan        : exclusive prefix of the counts over blocks (one block of
//                 threads per expert) and over experts -> expert_offset.
//   place_gather: every block re-walks its slots in order, ranks them inside
//                 their expert with warp match/popc, writes
//                 invert_permutation and copies each token row once from X to
//                 its k destinations.
// Decode-size batches (<= 1024 tokens, <= 64 experts), one launch:
//   select_small: every block repeats the routing of all tokens and derives the
//                 positions of its own slots from warp ballots.
//   route_select: the same with the router logits (x . W_gate^T) computed in the
//                 kernel and one bounded, self-resetting grid-wide barrier.
#include "common.cuh"

namespace pmx {
namespace {

constexpr int kMaxSlotsPerBlock = 2048;

// Scratch of pmx_moe_select_static: lives in the library's device image, so
// every GPU that loads the library holds these bytes until the process exits.
// In host code the name below is only a handle for cudaGetSymbolAddress; the
// kernels are always given the address that call returns.
static __device__ __align__(256) unsigned char g_select_static_scratch[PMX_MOE_SELECT_STATIC_SCRATCH_BYTES];

// Order-preserving map of a score to an unsigned key: -0 == +0, NaN on top.
__device__ __forceinline__ uint32_t score_key(float s) {
  if (s != s) return 0xFFFFFFFFu;
  if (s == 0.0f) s = 0.0f;
  uint32_t u = __float_as_uint(s);
  return (u >> 31) ? ~u : (u | 0x80000000u);
}

template <typename T>
__global__ void route_count_kernel(const T* scores, int64_t T_tokens, int E, int k,
                                   int tpb, T* __restrict__ weights, int* __restrict__ ids,
                                   int* __restrict__ block_counts) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int hist[];  // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int64_t t0 = (int64_t)blockIdx.x * tpb;
  for (int tl = warp; tl < tpb; tl += nwarps) {
    const int64_t t = t0 + tl;
    if (t >= T_tokens) break;
    const T* row = scores + t * E;
    // composite key: score key in the high word, inverted expert index in the
    // low word, so that a plain maximum prefers the lower index among equals
    // and every expert has a distinct key.
    unsigned long long prev = ~0ull;
    float vmax = 0.f, denom = 0.f, myexp = 0.f;
    int mysel = -1;
    for (int j = 0; j < k; ++j) {
      unsigned long long best = 0ull;
      for (int e = lane; e < E; e += 32) {
        unsigned long long key =
            ((unsigned long long)score_key(Elem<T>::to_f(row[e])) << 32) | (uint32_t)(0x7FFFFFFF - e);
        if (key < prev && key > best) best = key;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        best = other > best ? other : best;
      }
      prev = best;
      const int e_sel = 0x7FFFFFFF - (int)(uint32_t)(best & 0xFFFFFFFFull);
      const float v = Elem<T>::to_f(row[e_sel]);
      if (j == 0) vmax = v;
      const float ex = expf(v - vmax);
      denom += ex;
      if (lane == j) {  // lane j keeps slot j (k <= 32)
        myexp = ex;
        mysel = e_sel;
      }
    }
    if (lane < k) {
      weights[t * k + lane] = Elem<T>::from_f(myexp / denom);
      ids[t * k + lane] = mysel;
      atomicAdd(&hist[mysel], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) block_counts[(int64_t)e * gridDim.x + blockIdx.x] = hist[e];
}

// block_counts[E][nblk] -> exclusive prefix over blocks in place (one block of
// threads per expert, coalesced); the last block to finish turns the per-expert
// totals into expert_offset.
__global__ void scan_kernel(int* __restrict__ block_counts, int nblk, int E, int* __restrict__ totals,
                            unsigned int* __restrict__ ticket, int64_t* __restrict__ expert_offset) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int warp_sum[32];
  __shared__ int carry;
  __shared__ bool last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int e = blockIdx.x;
  int* col = block_counts + (int64_t)e * nblk;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int b0 = 0; b0 < nblk; b0 += blockDim.x) {
    const int b = b0 + threadIdx.x;
    const int v = b < nblk ? col[b] : 0;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (lane >= o) incl += n;
    }
    if (lane == 31) warp_sum[warp] = incl;
    __syncthreads();
    int before = carry;
    for (int w = 0; w < warp; ++w) before += warp_sum[w];
    if (b < nblk) col[b] = before + incl - v;
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry = before + incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    totals[e] = carry;
    __threadfence();
    last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (last) {
    __threadfence();
    if (threadIdx.x == 0) {
      int64_t acc = 0;
      for (int i = 0; i < E; ++i) {
        expert_offset[i] = acc;
        acc += *reinterpret_cast<volatile int*>(&totals[i]);
      }
      expert_offset[E] = acc;
      *ticket = 0;
    }
  }
  (void)nwarps;
}

template <typename T, bool VEC>
__global__ void place_gather_kernel(const T* x, const int* ids,
                                    const int* block_base,
                                    const int64_t* expert_offset, int64_t T_tokens,
                                    int64_t H, int E, int k, int tpb, T* __restrict__ xp,
                                    int64_t* __restrict__ inv) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int sm[];
  int* cursor = sm;      // [E] next row of each expert for this block
  int* pos = sm + E;     // [tpb*k] destination row of each slot of this block
  const int64_t t0 = (int64_t)blockIdx.x * tpb;
  const int ntok = (int)min((int64_t)tpb, T_tokens - t0);
  const int nslots = ntok * k;
  const int64_t slot0 = t0 * k;
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    cursor[e] = (int)expert_offset[e] + block_base[(int64_t)e * gridDim.x + blockIdx.x];
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    for (int g = 0; g < nslots; g += 32) {
      const int s = g + lane;
      const bool valid = s < nslots;
      const int e = valid ? ids[slot0 + s] : -1 - lane;
      const unsigned peers = __match_any_sync(0xFFFFFFFFu, e);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      int p = 0;
      if (valid) p = cursor[e] + rank;
      __syncwarp();
      if (valid && rank == __popc(peers) - 1) cursor[e] = p + 1;
      __syncwarp();
      if (valid) {
        pos[s] = p;
        inv[slot0 + s] = p;
      }
    }
  }
  __syncthreads();
  if (VEC) {
    const int chunks = (int)(H * sizeof(T) / 16);
    const uint4* src = reinterpret_cast<const uint4*>(x + t0 * H);
    uint4* dst = reinterpret_cast<uint4*>(xp);
    const int total = ntok * chunks;
    // four independent 16-byte loads in flight per thread before the stores
    for (int i0 = threadIdx.x; i0 < total; i0 += 4 * blockDim.x) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < total) v[u] = __ldcg(src + i);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < total) {
          const int tl = i / chunks, c = i - tl * chunks;
          for (int j = 0; j < k; ++j) dst[(int64_t)pos[tl * k + j] * chunks + c] = v[u];
        }
      }
    }
  } else {
    const int64_t total = (int64_t)ntok * H;
    for (int64_t i = threadIdx.x; i < total; i += blockDim.x) {
      const int tl = (int)(i / H);
      const int64_t c = i - (int64_t)tl * H;
      const T v = x[(t0 + tl) * H + c];
      for (int j = 0; j < k; ++j) xp[(int64_t)pos[tl * k + j] * H + c] = v;
    }
  }
}

// ---- single-launch variant for decode-size batches ---------------------------
// Every block repeats the routing of ALL tokens (a thread per token, cheap for
// T <= 1024) instead of exchanging counts through global memory, then gathers
// only its own tokens.  Because the k experts of one token are distinct, the
// stable position of slot (t, j) with expert e is
//     expert_offset[e] + number of tokens t' < t that selected e,
// which comes from warp ballots: B[g][e] = ballot over the 32 tokens of group g
// of "token selected e".
constexpr int kSmallMaxTokens = 1024;
constexpr int kSmallMaxExperts = 64;

template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
select_small_kernel(const T* x, const T* scores, int Tn, int64_t H, int E,
                    int k, int tpb, T* __restrict__ xp, T* __restrict__ weights,
                    int64_t* __restrict__ inv, int64_t* __restrict__ expert_offset) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ unsigned int sm_small[];
  const int groups = (Tn + 31) / 32;
  unsigned int* ballots = sm_small;                                     // [groups][E]
  int* group_base = reinterpret_cast<int*>(ballots + groups * E);       // [groups][E] tokens of earlier groups
  int* offs = group_base + groups * E;                                   // [E+1]
  short* ids = reinterpret_cast<short*>(offs + E + 1);                   // [groups*32][k]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const bool writer = blockIdx.x == 0;   // block 0 also writes the small outputs

  for (int g = warp; g < groups; g += nwarps) {
    const int t = g * 32 + lane;
    unsigned long long mask = 0ull;      // experts selected by this token
    if (t < Tn) {
      const T* row = scores + (int64_t)t * E;
      unsigned long long prev = ~0ull;
      float vmax = 0.f, denom = 0.f;
      for (int j = 0; j < k; ++j) {
        unsigned long long best = 0ull;
        for (int e = 0; e < E; ++e) {
          const unsigned long long key =
              ((unsigned long long)score_key(Elem<T>::to_f(row[e])) << 32) | (uint32_t)(0x7FFFFFFF - e);
          if (key < prev && key > best) best = key;
        }
        prev = best;
        const int e_sel = 0x7FFFFFFF - (int)(uint32_t)(best & 0xFFFFFFFFull);
        ids[t * k + j] = (short)e_sel;
        mask |= 1ull << e_sel;
        const float v = Elem<T>::to_f(row[e_sel]);
        if (j == 0) vmax = v;
        denom += expf(v - vmax);
      }
      if (writer) {
        for (int j = 0; j < k; ++j) {
          const float v = Elem<T>::to_f(row[ids[t * k + j]]);
          weights[(int64_t)t * k + j] = Elem<T>::from_f(expf(v - vmax) / denom);
        }
      }
    }
    for (int e = 0; e < E; ++e) {
      const unsigned int b = __ballot_sync(0xFFFFFFFFu, (mask >> e) & 1ull);
      if (lane == 0) ballots[g * E + e] = b;
    }
  }
  __syncthreads();
  // per expert: tokens in earlier groups, total, then offsets
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int g = 0; g < groups; ++g) {
      group_base[g * E + e] = run;
      run += __popc(ballots[g * E + e]);
    }
    offs[e + 1] = run;   // totals for now
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      const int c = offs[e + 1];
      offs[e] = acc;
      acc += c;
    }
    offs[E] = acc;
  }
  __syncthreads();
  if (writer) {
    for (int e = threadIdx.x; e <= E; e += blockDim.x) expert_offset[e] = offs[e];
    for (int s = threadIdx.x; s < Tn * k; s += blockDim.x) {
      const int t = s / k, e = ids[s];
      const int g = t >> 5, l = t & 31;
      inv[s] = offs[e] + group_base[g * E + e] + __popc(ballots[g * E + e] & ((1u << l) - 1u));
    }
  }
  // gather this block's tokens
  const int t0 = blockIdx.x * tpb;
  const int ntok = min(tpb, Tn - t0);
  if (ntok <= 0) return;
  int* pos = reinterpret_cast<int*>(ids + (size_t)groups * 32 * k);   // [tpb*k] rows of my slots
  for (int i = threadIdx.x; i < ntok * k; i += blockDim.x) {
    const int t = t0 + i / k, e = ids[t0 * k + i];
    const int g = t >> 5, l = t & 31;
    pos[i] = offs[e] + group_base[g * E + e] + __popc(ballots[g * E + e] & ((1u << l) - 1u));
  }
  __syncthreads();
  if (VEC) {
    const int chunks = (int)(H * sizeof(T) / 16);
    const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)t0 * H);
    uint4* dst = reinterpret_cast<uint4*>(xp);
    for (int i = threadIdx.x; i < ntok * chunks; i += blockDim.x) {
      const int tl = i / chunks, c = i - tl * chunks;
      const uint4 v = __ldcg(src + (int64_t)tl * chunks + c);
      for (int j = 0; j < k; ++j) dst[(int64_t)pos[tl * k + j] * chunks + c] = v;
    }
  } else {
    for (int64_t i = threadIdx.x; i < (int64_t)ntok * H; i += blockDim.x) {
      const int tl = (int)(i / H);
      const int64_t c = i - (int64_t)tl * H;
      const T v = x[(int64_t)(t0 + tl) * H + c];
      for (int j = 0; j < k; ++j) xp[(int64_t)pos[tl * k + j] * H + c] = v;
    }
  }
}

bool select_small_applies(int64_t T, int E, int k) {
  return T <= kSmallMaxTokens && E <= kSmallMaxExperts && k <= 32;
}

template <typename T>
int run_select_small(const void* x, const void* scores, void* xp, void* w, int64_t* inv, int64_t* off,
                     int64_t Tn, int64_t H, int E, int k, cudaStream_t s) {
  const int groups = (int)ceil_div(Tn, 32);
  // tokens per block: spread the row copies over the SMs
  int tpb = (int)ceil_div(Tn, (int64_t)sm_count());
  if (tpb < 1) tpb = 1;
  const int nblk = (int)ceil_div(Tn, tpb);
  size_t smem = (size_t)groups * E * 8 + (size_t)(E + 1) * 4 + (size_t)groups * 32 * k * 2;
  smem = ((smem + 3) & ~(size_t)3) + (size_t)tpb * k * 4 + 16;
  const bool vec = (H * sizeof(T)) % 16 == 0 && aligned16(x) && aligned16(xp);
  auto kern = vec ? select_small_kernel<T, true> : select_small_kernel<T, false>;
  if (smem > 48 * 1024) PMX_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  return launch_pdl_k(kern, dim3(nblk), dim3(256), smem, s, reinterpret_cast<const T*>(x),
                      reinterpret_cast<const T*>(scores), (int)Tn, H, E, k, tpb, reinterpret_cast<T*>(xp),
                      reinterpret_cast<T*>(w), inv, off);
}

// ---- router gate + select in one launch ---------------------------------------
// For decode-size batches the router logits (Linear.forward, Linear.py:24-33,
// called at Model.py:188) are computed by the same kernel that routes: each
// block computes the E logits of its own tokens (fp32 accumulation, one rounding
// to T1 -- the scores the reference would hand to moe_select), picks their top-k
// and publishes one 64-bit expert mask per token; after a grid-wide barrier
// (bounded spin on a generation word; the grid has at most one block per SM, so
// all blocks are resident together) every block derives the stable positions of its own slots from the
// masks of all tokens and gathers its rows.  The grid has at most one block per SM.
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// NORM: the rows routed are RMSNorm(x (+ skip)) * norm_w (SkipRMSNorm.forward,
// RMSNorm.py:42-56, the ffn_norm of Model.py:261): each block normalises its own tokens
// into shared memory first, writes the residual stream (skip_out) and then computes
// logits from, and gathers, the normalised rows.
struct NormArgs {
  const void* skip;      // [T,H] or null
  const void* weight;    // [H]
  void* skip_out;        // [T,H] (required when skip is given)
  float eps;
};

__device__ __forceinline__ unsigned long long route_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

template <typename T, bool NORM>
__global__ void __launch_bounds__(256)
route_select_kernel(const T* x, const T* wr, int Tn, int64_t H, int E, int k,
                    int tpb, T* __restrict__ scores, T* __restrict__ xp, T* __restrict__ weights,
                    int64_t* __restrict__ inv, int64_t* __restrict__ expert_offset,
                    unsigned long long* __restrict__ masks, unsigned int* __restrict__ counter,
                    int* __restrict__ status, NormArgs norm, unsigned long long wait_ns,
                    unsigned long long* stamps) {
  extern __shared__ unsigned int sm_rs[];
  const int groups = (Tn + 31) / 32;
  unsigned int* ballots = sm_rs;                                        // [groups][E]
  int* group_base = reinterpret_cast<int*>(ballots + groups * E);      // [groups][E]
  int* offs = group_base + groups * E;                                  // [E+1]
  float* logit = reinterpret_cast<float*>(offs + E + 1);                // [tpb][E]
  int* my_ids = reinterpret_cast<int*>(logit + tpb * E);                // [tpb][k]
  int* pos = my_ids + tpb * k;                                          // [tpb][k]
  float* partial = reinterpret_cast<float*>(pos + tpb * k);             // [warps][E]
  // NORM: normalised rows of my tokens, 16-byte aligned behind the arrays above
  uint4* rows = reinterpret_cast<uint4*>((reinterpret_cast<uintptr_t>(partial + 8 * E) + 15) & ~uintptr_t(15));
  __shared__ int s_abort;
  __shared__ float s_norm_sum[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int t0 = blockIdx.x * tpb;
  const int ntok = max(0, min(tpb, Tn - t0));
  constexpr int V = kVec<T>;
  const int chunks = (int)(H / V);
  if (threadIdx.x == 0) s_abort = 0;
  if (stamps && threadIdx.x == 0 && blockIdx.x < 160) stamps[blockIdx.x * 8 + 0] = route_ns();
  // The dependent kernel may read x while this one runs (the dense gate/up projection does):
  // it is released only after this kernel's own predecessors, which produced x, are complete.
  pdl_wait();   // x (and skip) come from the kernel in front of this one
  pdl_launch_dependents();
  if (stamps && threadIdx.x == 0 && blockIdx.x < 160) stamps[blockIdx.x * 8 + 1] = route_ns();

  // A0. (NORM) normalise my tokens into shared memory
  if (NORM) {
    const T* nw = reinterpret_cast<const T*>(norm.weight);
    for (int tl = 0; tl < ntok; ++tl) {
      const uint4* xr = reinterpret_cast<const uint4*>(x + (int64_t)(t0 + tl) * H);
      const uint4* sr = norm.skip ? reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(norm.skip) + (int64_t)(t0 + tl) * H) : nullptr;
      uint4* so = norm.skip ? reinterpret_cast<uint4*>(reinterpret_cast<T*>(norm.skip_out) + (int64_t)(t0 + tl) * H) : nullptr;
      uint4* row = rows + (size_t)tl * chunks;
      float acc = 0.f;
      for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        float a[V];
        unpack16<T>(__ldcg(xr + c), a);
        if (sr) {
          float b[V];
          unpack16<T>(__ldcg(sr + c), b);
#pragma unroll
          for (int v = 0; v < V; ++v) a[v] = Elem<T>::to_f(Elem<T>::from_f(a[v] + b[v]));
          so[c] = pack16<T>(a);
        }
#pragma unroll
        for (int v = 0; v < V; ++v) acc = fmaf(a[v], a[v], acc);
        row[c] = pack16<T>(a);          // the (rounded) sum, scaled in place below
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
      if (lane == 0) s_norm_sum[warp] = acc;
      __syncthreads();
      float tot = 0.f;
      for (int w = 0; w < nwarps; ++w) tot += s_norm_sum[w];
      const float scale = rsqrtf(tot / (float)H + norm.eps);
      for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        float a[V], wv[V];
        unpack16<T>(row[c], a);
        unpack16<T>(__ldg(reinterpret_cast<const uint4*>(nw) + c), wv);
#pragma unroll
        for (int v = 0; v < V; ++v) a[v] = Elem<T>::to_f(Elem<T>::from_f(a[v] * scale)) * wv[v];
        row[c] = pack16<T>(a);
      }
      __syncthreads();
    }
  }
  // A1. logits of my tokens.  The warps split the hidden dimension; every lane
  // keeps 8 experts' partial dot products, so one pass issues 9 independent
  // 16-byte loads per lane.  Partial sums meet in shared memory.
  for (int tl = 0; tl < ntok; ++tl) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (int64_t)(t0 + tl) * H);
    for (int e0 = 0; e0 < E; e0 += 8) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        float a[V];
        unpack16<T>(NORM ? rows[(size_t)tl * chunks + c] : __ldcg(xr + c), a);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (e0 + j < E) {
            float b[V];
            unpack16<T>(__ldg(reinterpret_cast<const uint4*>(wr + (int64_t)(e0 + j) * H) + c), b);
#pragma unroll
            for (int v = 0; v < V; ++v) acc[j] = fmaf(a[v], b[v], acc[j]);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[j] += __shfl_xor_sync(0xFFFFFFFFu, acc[j], o);
        if (lane == 0 && e0 + j < E) partial[warp * E + e0 + j] = acc[j];
      }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      float sum = 0.f;
      for (int w = 0; w < nwarps; ++w) sum += partial[w * E + e];
      const T r = Elem<T>::from_f(sum);
      scores[(int64_t)(t0 + tl) * E + e] = r;
      logit[tl * E + e] = Elem<T>::to_f(r);
    }
    __syncthreads();
  }
  // A2. top-k of my tokens (a thread per token), softmax weights, expert mask
  if (threadIdx.x < ntok) {
    const int tl = threadIdx.x, t = t0 + tl;
    const float* row = logit + tl * E;
    unsigned long long prev = ~0ull, mask = 0ull;
    float vmax = 0.f, denom = 0.f;
    for (int j = 0; j < k; ++j) {
      unsigned long long best = 0ull;
      for (int e = 0; e < E; ++e) {
        const unsigned long long key = ((unsigned long long)score_key(row[e]) << 32) | (uint32_t)(0x7FFFFFFF - e);
        if (key < prev && key > best) best = key;
      }
      prev = best;
      const int e_sel = 0x7FFFFFFF - (int)(uint32_t)(best & 0xFFFFFFFFull);
      my_ids[tl * k + j] = e_sel;
      mask |= 1ull << e_sel;
      if (j == 0) vmax = row[e_sel];
      denom += expf(row[e_sel] - vmax);
    }
    for (int j = 0; j < k; ++j)
      weights[(int64_t)t * k + j] = Elem<T>::from_f(expf(row[my_ids[tl * k + j]] - vmax) / denom);
    masks[t] = mask;
  }
  // grid-wide barrier: everybody's masks are in global memory.  Sense-reversing and
  // self-resetting (the last block to arrive clears the count and advances the
  // generation), so the two words only have to be zero once, before the first call.
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int* generation = counter + 1;
    const unsigned int gen0 = ld_acquire_gpu(generation);   // cannot advance before this block arrives
    __threadfence();
    if (atomicAdd(counter, 1u) == gridDim.x - 1) {
      *reinterpret_cast<volatile unsigned int*>(counter) = 0u;
      __threadfence();
      st_release_gpu(generation, gen0 + 1u);
    } else {
      unsigned long long t_start = 0;
      unsigned int it = 0;
      while (ld_acquire_gpu(generation) == gen0) {
        if ((++it & 1023u) == 0u) {
          unsigned long long now;
          asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
          if (t_start == 0) t_start = now;
          if (now - t_start > wait_ns) {   // give up, record it
            s_abort = 1;
            atomicCAS(status, 0, 2);
            break;
          }
        }
      }
    }
  }
  __syncthreads();
  if (s_abort) return;
  if (stamps && threadIdx.x == 0 && blockIdx.x < 160) stamps[blockIdx.x * 8 + 2] = route_ns();

  // B. ballots over all tokens from the masks
  for (int g = warp; g < groups; g += nwarps) {
    const int t = g * 32 + lane;
    const unsigned long long m = t < Tn ? __ldcg(masks + t) : 0ull;
    for (int e = 0; e < E; ++e) {
      const unsigned int b = __ballot_sync(0xFFFFFFFFu, (m >> e) & 1ull);
      if (lane == 0) ballots[g * E + e] = b;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int g = 0; g < groups; ++g) {
      group_base[g * E + e] = run;
      run += __popc(ballots[g * E + e]);
    }
    offs[e + 1] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      const int c = offs[e + 1];
      offs[e] = acc;
      acc += c;
    }
    offs[E] = acc;
  }
  __syncthreads();
  if (blockIdx.x == 0)
    for (int e = threadIdx.x; e <= E; e += blockDim.x) expert_offset[e] = offs[e];
  for (int i = threadIdx.x; i < ntok * k; i += blockDim.x) {
    const int t = t0 + i / k, e = my_ids[i];
    const int g = t >> 5, l = t & 31;
    const int p = offs[e] + group_base[g * E + e] + __popc(ballots[g * E + e] & ((1u << l) - 1u));
    pos[i] = p;
    inv[(int64_t)t0 * k + i] = p;
  }
  __syncthreads();
  if (stamps && threadIdx.x == 0 && blockIdx.x < 160) stamps[blockIdx.x * 8 + 6] = route_ns();
  // C. gather my tokens (not wanted by callers that feed the un-permuted tokens to the experts)
  if (xp == nullptr) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)t0 * H);
  uint4* dst = reinterpret_cast<uint4*>(xp);
  for (int i = threadIdx.x; i < ntok * chunks; i += blockDim.x) {
    const int tl = i / chunks, c = i - tl * chunks;
    const uint4 v = NORM ? rows[i] : __ldcg(src + (int64_t)tl * chunks + c);
    for (int j = 0; j < k; ++j) dst[(int64_t)pos[tl * k + j] * chunks + c] = v;
  }
}

struct RouteSelectGeometry {
  int tpb, nblk;
  size_t smem;
};

bool route_select_geometry(int64_t T, int64_t H, int E, int k, int dtype, RouteSelectGeometry* g,
                           bool with_norm = false) {
  const int vec = dtype == PMX_DTYPE_F32 ? 4 : 8;
  if (T <= 0 || T > kSmallMaxTokens || E <= 0 || E > kSmallMaxExperts || k <= 0 || k > 32 || k > E || H % vec) return false;
  const int sms = sm_count();
  g->tpb = (int)ceil_div(T, (int64_t)sms);
  g->nblk = (int)ceil_div(T, g->tpb);
  const int groups = (int)ceil_div(T, 32);
  g->smem = ((size_t)groups * E * 2 + (E + 1) + (size_t)g->tpb * E + 2 * (size_t)g->tpb * k + 8 * (size_t)E) * 4 + 16;
  if (with_norm) g->smem += 16 + (size_t)g->tpb * H * (dtype == PMX_DTYPE_F32 ? 4 : 2);
  return g->nblk <= sms && g->smem <= 200 * 1024;
}

// ---- one launch for large batches (up to 64 experts) ----------------------------
// Every block owns `tpb` consecutive tokens: it routes them (a thread per token, the
// block's scores staged in shared memory), leaves its per-expert counts in global
// memory, meets the other blocks at one bounded grid-wide barrier (at most one block per
// SM, so all are resident), adds up the counts of the blocks in front of it, and then
// places and gathers its own rows.  Positions only depend on the scores (no atomics
// decide an order), so every tensor-parallel rank computes the same permutation.
constexpr int kWideChunk = 256;          // tokens routed per pass (one per thread of the first 8 warps)
constexpr int kWideThreads = 1024;       // one block per SM: the row copies need many loads in flight
constexpr int kWideMaxTokensPerBlock = 1024;

template <typename T, bool VEC>
__global__ void __launch_bounds__(kWideThreads)
select_wide_kernel(const T* x, const T* scores, int64_t Tn, int64_t H, int E, int k,
                   int tpb, T* __restrict__ xp, T* __restrict__ weights, int64_t* __restrict__ inv,
                   int64_t* __restrict__ expert_offset, unsigned int* __restrict__ barrier,
                   int* __restrict__ block_counts, int* __restrict__ status, unsigned long long wait_ns) {
  extern __shared__ unsigned int sm_wide[];
  const int groups = (tpb + 31) / 32;
  unsigned int* ballots = sm_wide;                                       // [groups][E]
  int* group_base = reinterpret_cast<int*>(ballots + groups * E);       // [groups][E] tokens of earlier groups
  int* offs = group_base + groups * E;                                   // [E] first row of this block's slots
  int* totals = offs + E;                                                // [E] rows of each expert, all blocks
  int* pos = totals + E;                                                 // [tpb*k]
  float* srow = reinterpret_cast<float*>(pos + tpb * k);                 // [kWideChunk][E+1] staged scores
  short* ids = reinterpret_cast<short*>(srow + kWideChunk * (E + 1));    // [groups*32][k]
  __shared__ int s_abort;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int64_t t0 = (int64_t)blockIdx.x * tpb;
  const int ntok = (int)min((int64_t)tpb, Tn - t0);
  if (threadIdx.x == 0) s_abort = 0;
  pdl_launch_dependents();
  pdl_wait();

  // A. routing of my tokens, kWideChunk at a time
  for (int c0 = 0; c0 < groups * 32; c0 += kWideChunk) {
    const int cn = min(kWideChunk, ntok - c0);       // may be <= 0 for the padding of the last group
    __syncthreads();
    for (int i = threadIdx.x; i < cn * E; i += blockDim.x) {
      const int tl = i / E, e = i - tl * E;
      srow[tl * (E + 1) + e] = Elem<T>::to_f(scores[(t0 + c0) * E + i]);
    }
    __syncthreads();
    const int tl = c0 + threadIdx.x;                 // token of this thread (its warp = one group)
    if (threadIdx.x < kWideChunk && tl < groups * 32) {
      unsigned long long mask = 0ull;
      if (tl < ntok) {
        const float* row = srow + threadIdx.x * (E + 1);
        unsigned long long prev = ~0ull;
        float vmax = 0.f, denom = 0.f;
        for (int j = 0; j < k; ++j) {
          unsigned long long best = 0ull;
          for (int e = 0; e < E; ++e) {
            const unsigned long long key = ((unsigned long long)score_key(row[e]) << 32) | (uint32_t)(0x7FFFFFFF - e);
            if (key < prev && key > best) best = key;
          }
          prev = best;
          const int e_sel = 0x7FFFFFFF - (int)(uint32_t)(best & 0xFFFFFFFFull);
          ids[tl * k + j] = (short)e_sel;
          mask |= 1ull << e_sel;
          if (j == 0) vmax = row[e_sel];
          denom += expf(row[e_sel] - vmax);
        }
        for (int j = 0; j < k; ++j)
          weights[(t0 + tl) * k + j] = Elem<T>::from_f(expf(row[ids[tl * k + j]] - vmax) / denom);
      }
      const int g = tl >> 5;
      for (int e = 0; e < E; ++e) {
        const unsigned int b = __ballot_sync(0xFFFFFFFFu, (mask >> e) & 1ull);
        if (lane == 0) ballots[g * E + e] = b;
      }
    }
  }
  __syncthreads();
  // B. per expert: tokens in earlier groups of this block, and the block's count
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int g = 0; g < groups; ++g) {
      group_base[g * E + e] = run;
      run += __popc(ballots[g * E + e]);
    }
    block_counts[(int64_t)e * gridDim.x + blockIdx.x] = run;
  }
  // C. grid-wide barrier (the count word is cleared by a memset node in front of the launch)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(barrier, 1u);
    unsigned long long t_start = 0;
    unsigned int it = 0;
    while (ld_acquire_gpu(barrier) < gridDim.x) {
      if ((++it & 1023u) == 0u) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        if (t_start == 0) t_start = now;
        if (now - t_start > wait_ns) {
          s_abort = 1;
          atomicCAS(status, 0, 2);
          break;
        }
      }
    }
  }
  __syncthreads();
  if (s_abort) return;
  // D. rows of every expert in the blocks in front of me, and in all blocks (a warp per expert)
  for (int e = warp; e < E; e += nwarps) {
    int before = 0, total = 0;
    for (int b = lane; b < (int)gridDim.x; b += 32) {
      const int c = __ldcg(block_counts + (int64_t)e * gridDim.x + b);
      total += c;
      if (b < (int)blockIdx.x) before += c;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      before += __shfl_xor_sync(0xFFFFFFFFu, before, o);
      total += __shfl_xor_sync(0xFFFFFFFFu, total, o);
    }
    if (lane == 0) {
      offs[e] = before;
      totals[e] = total;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      if (blockIdx.x == 0) expert_offset[e] = acc;
      offs[e] += acc;
      acc += totals[e];
    }
    if (blockIdx.x == 0) expert_offset[E] = acc;
  }
  __syncthreads();
  // E. stable positions of my slots
  for (int i = threadIdx.x; i < ntok * k; i += blockDim.x) {
    const int tl = i / k, e = ids[i];
    const int g = tl >> 5, l = tl & 31;
    const int p = offs[e] + group_base[g * E + e] + __popc(ballots[g * E + e] & ((1u << l) - 1u));
    pos[i] = p;
    inv[t0 * k + i] = p;
  }
  __syncthreads();
  // F. gather my rows: each token row is read once and written to its k destinations
  if (VEC) {
    const int chunks = (int)(H * sizeof(T) / 16);
    const uint4* src = reinterpret_cast<const uint4*>(x + t0 * H);
    uint4* dst = reinterpret_cast<uint4*>(xp);
    const int total = ntok * chunks;
    for (int i0 = threadIdx.x; i0 < total; i0 += 4 * blockDim.x) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < total) v[u] = __ldcg(src + i);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < total) {
          const int tl = i / chunks, c = i - tl * chunks;
          for (int j = 0; j < k; ++j) dst[(int64_t)pos[tl * k + j] * chunks + c] = v[u];
        }
      }
    }
  } else {
    const int64_t total = (int64_t)ntok * H;
    for (int64_t i = threadIdx.x; i < total; i += blockDim.x) {
      const int tl = (int)(i / H);
      const int64_t c = i - (int64_t)tl * H;
      const T v = x[(t0 + tl) * H + c];
      for (int j = 0; j < k; ++j) xp[(int64_t)pos[tl * k + j] * H + c] = v;
    }
  }
}

struct WideGeometry {
  int tpb, nblk;
  size_t smem;
};

// One block per SM at most (the blocks wait for one another), at least 32 tokens each.
bool select_wide_geometry(int64_t T, int E, int k, WideGeometry* g) {
  if (E > kSmallMaxExperts || k > 32) return false;
  const int sms = sm_count();
  int64_t tpb = ceil_div(T, (int64_t)sms);
  tpb = ceil_div(tpb, 32) * 32;
  if (tpb > kWideMaxTokensPerBlock) return false;
  g->tpb = (int)tpb;
  g->nblk = (int)ceil_div(T, tpb);
  const size_t groups = (size_t)tpb / 32;
  g->smem = (groups * E * 2 + 2 * (size_t)E + (size_t)tpb * k + (size_t)kWideChunk * (E + 1)) * 4 +
            groups * 32 * k * 2 + 16;
  return g->nblk <= sms && g->smem <= 200 * 1024;
}

struct SelectGeometry {
  int tpb;
  int nblk;
  size_t ids_bytes;
  size_t counts_bytes;
};

SelectGeometry select_geometry(int64_t T, int E, int k) {
  SelectGeometry g;
  // enough blocks to cover the SMs twice for small T, up to 16 tokens per block
  int64_t tpb = T / 296;
  if (tpb < 1) tpb = 1;
  if (tpb > 16) tpb = 16;
  if (tpb * k > kMaxSlotsPerBlock) tpb = kMaxSlotsPerBlock / k > 0 ? kMaxSlotsPerBlock / k : 1;
  g.tpb = (int)tpb;
  g.nblk = (int)ceil_div(T, tpb);
  g.ids_bytes = (size_t)ceil_div(T * k * 4, 16) * 16;
  // per-block counts [E][nblk], then per-expert totals [E] and the scan's ticket word
  g.counts_bytes = (size_t)ceil_div(((int64_t)g.nblk * E + E + 4) * 4, 16) * 16;
  return g;
}

template <typename T>
int run_select(const void* x, const void* scores, void* xp, void* w, int64_t* inv, int64_t* off,
               int64_t Tn, int64_t H, int E, int k, void* ws, cudaStream_t s) {
  if (select_small_applies(Tn, E, k)) return run_select_small<T>(x, scores, xp, w, inv, off, Tn, H, E, k, s);
  WideGeometry wg;
  if (select_wide_geometry(Tn, E, k, &wg)) {
    // scratch: 16 bytes of barrier / status words, then the per-block counts [E][blocks]
    unsigned int* barrier = reinterpret_cast<unsigned int*>(ws);
    int* status = reinterpret_cast<int*>(ws) + 2;
    int* block_counts = reinterpret_cast<int*>(ws) + 4;
    PMX_CUDA_OK(cudaMemsetAsync(ws, 0, 16, s));
    const bool vec = (H * sizeof(T)) % 16 == 0 && aligned16(x) && aligned16(xp);
    auto kern = vec ? select_wide_kernel<T, true> : select_wide_kernel<T, false>;
    if (wg.smem > 48 * 1024) PMX_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wg.smem));
    return launch_pdl_k(kern, dim3(wg.nblk), dim3(kWideThreads), wg.smem, s, reinterpret_cast<const T*>(x),
                        reinterpret_cast<const T*>(scores), Tn, H, E, k, wg.tpb, reinterpret_cast<T*>(xp),
                        reinterpret_cast<T*>(w), inv, off, barrier, block_counts, status, 1000000000ull);
  }
  const SelectGeometry g = select_geometry(Tn, E, k);
  int* ids = reinterpret_cast<int*>(ws);
  int* counts = reinterpret_cast<int*>(reinterpret_cast<char*>(ws) + g.ids_bytes);
  const int route_threads = 32 * (g.tpb < 8 ? g.tpb : 8);
  int st = launch_pdl_k(route_count_kernel<T>, dim3(g.nblk), dim3(route_threads), E * sizeof(int), s,
                        reinterpret_cast<const T*>(scores), Tn, E, k, g.tpb, reinterpret_cast<T*>(w), ids, counts);
  if (st != PMX_OK) return st;
  int* totals = counts + (int64_t)g.nblk * E;
  unsigned int* ticket = reinterpret_cast<unsigned int*>(totals + E);
  PMX_CUDA_OK(cudaMemsetAsync(ticket, 0, sizeof(unsigned int), s));
  st = launch_pdl_k(scan_kernel, dim3(E), dim3(256), 0, s, counts, g.nblk, E, totals, ticket, off);
  if (st != PMX_OK) return st;
  const size_t sm_bytes = (size_t)(E + g.tpb * k) * sizeof(int);
  const bool vec = (H * sizeof(T)) % 16 == 0 && aligned16(x) && aligned16(xp);
  auto place = vec ? place_gather_kernel<T, true> : place_gather_kernel<T, false>;
  return launch_pdl_k(place, dim3(g.nblk), dim3(256), sm_bytes, s, reinterpret_cast<const T*>(x), ids, counts, off, Tn,
                      H, E, k, g.tpb, reinterpret_cast<T*>(xp), inv);
}

}  // namespace

size_t select_workspace_bytes(int64_t T, int E, int k) {
  if (T <= 0 || E <= 0 || k <= 0) return 0;
  const SelectGeometry g = select_geometry(T, E, k);
  return g.ids_bytes + g.counts_bytes;
}

int launch_select(const void* x, const void* scores, void* xp, void* w, int64_t* inv, int64_t* off,
                  int64_t T, int64_t H, int E, int k, int dtype, void* ws, size_t ws_bytes,
                  cudaStream_t s) {
  if (!x || !scores || !xp || !w || !inv || !off) return fail(PMX_ERR_INVALID_ARGUMENT, "moe_select: null pointer");
  if (T <= 0) return fail(PMX_ERR_INVALID_ARGUMENT, "moe_select: needs at least one token (T=%lld)", (long long)T);
  if (H <= 0 || E <= 0 || k <= 0) return fail(PMX_ERR_INVALID_ARGUMENT, "moe_select: H, E, k must be positive");
  if (k > E) return fail(PMX_ERR_INVALID_ARGUMENT, "moe_select: k=%d exceeds the number of experts %d", k, E);
  if (k > 32) return fail(PMX_ERR_UNSUPPORTED, "moe_select: at most 32 experts per token (k=%d)", k);
  if (E > 8192) return fail(PMX_ERR_UNSUPPORTED, "moe_select: at most 8192 experts");
  if (T * k >= (1ll << 31)) return fail(PMX_ERR_UNSUPPORTED, "moe_select: T*k must stay below 2^31");
  const size_t need = select_workspace_bytes(T, E, k);
  if (!ws || ws_bytes < need) return fail(PMX_ERR_WORKSPACE, "moe_select: workspace of %zu bytes needed, %zu given", need, ws_bytes);
  if (!aligned16(ws)) return fail(PMX_ERR_ALIGNMENT, "moe_select: workspace must be 16-byte aligned");
  switch (dtype) {
    case PMX_DTYPE_F16: return run_select<__half>(x, scores, xp, w, inv, off, T, H, E, k, ws, s);
    case PMX_DTYPE_BF16: return run_select<__nv_bfloat16>(x, scores, xp, w, inv, off, T, H, E, k, ws, s);
    case PMX_DTYPE_F32: return run_select<float>(x, scores, xp, w, inv, off, T, H, E, k, ws, s);
  }
  return fail(PMX_ERR_UNSUPPORTED, "moe_select: unknown dtype %d", dtype);
}

size_t route_select_workspace_bytes(int64_t T, int64_t H, int E, int k, int dtype) {
  RouteSelectGeometry g;
  if (!route_select_geometry(T, H, E, k, dtype, &g)) return 0;
  return 64 + (size_t)T * 8;   // counter + status words, then one expert mask per token
}

int launch_route_select_impl(const void* x, const void* wr, void* scores, void* xp, void* w, int64_t* inv,
                             int64_t* off, int64_t T, int64_t H, int E, int k, int dtype, void* ws,
                             size_t ws_bytes, cudaStream_t s, bool with_norm, NormArgs norm) {
  const char* name = with_norm ? "moe_norm_route_select" : "moe_route_select";
  if (!x || !wr || !scores || !w || !inv || !off) return fail(PMX_ERR_INVALID_ARGUMENT, "%s: null pointer", name);
  if (with_norm && (!norm.weight || (norm.skip && !norm.skip_out)))
    return fail(PMX_ERR_INVALID_ARGUMENT, "%s: norm weight missing, or skip given without skip_out", name);
  RouteSelectGeometry g;
  if (!route_select_geometry(T, H, E, k, dtype, &g, with_norm))
    return fail(PMX_ERR_UNSUPPORTED, "%s: covers 1..%d tokens, up to %d experts, k <= 32 and 16-byte rows (T=%lld E=%d k=%d H=%lld); use the stand-alone operators", name, kSmallMaxTokens, kSmallMaxExperts, (long long)T, E, k, (long long)H);
  const size_t need = route_select_workspace_bytes(T, H, E, k, dtype);
  if (!ws || ws_bytes < need) return fail(PMX_ERR_WORKSPACE, "%s: workspace of %zu bytes needed, %zu given", name, need, ws_bytes);
  if (!aligned16(ws) || !aligned16(x) || !aligned16(wr) || !aligned16(xp) ||
      (with_norm && (!aligned16(norm.weight) || !aligned16(norm.skip) || !aligned16(norm.skip_out))))
    return fail(PMX_ERR_ALIGNMENT, "%s: tensors and the workspace must be 16-byte aligned", name);
  unsigned int* counter = reinterpret_cast<unsigned int*>(ws);
  int* status = reinterpret_cast<int*>(ws) + 4;
  unsigned long long* masks = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(ws) + 64);
  int Tn = (int)T;
  unsigned long long wait_ns = 1000000000ull;   // 1 s
  unsigned long long* stamps = next_stamp_slot(1);
  void* args[] = {(void*)&x, (void*)&wr, (void*)&Tn, (void*)&H, (void*)&E, (void*)&k, (void*)&g.tpb, (void*)&scores,
                  (void*)&xp, (void*)&w, (void*)&inv, (void*)&off, (void*)&masks, (void*)&counter, (void*)&status,
                  (void*)&norm, (void*)&wait_ns, (void*)&stamps};
  const void* kern = nullptr;
  switch (dtype) {
    case PMX_DTYPE_F16: kern = with_norm ? (const void*)route_select_kernel<__half, true> : (const void*)route_select_kernel<__half, false>; break;
    case PMX_DTYPE_BF16: kern = with_norm ? (const void*)route_select_kernel<__nv_bfloat16, true> : (const void*)route_select_kernel<__nv_bfloat16, false>; break;
    case PMX_DTYPE_F32: kern = with_norm ? (const void*)route_select_kernel<float, true> : (const void*)route_select_kernel<float, false>; break;
    default: return fail(PMX_ERR_UNSUPPORTED, "%s: unknown dtype %d", name, dtype);
  }
  if (g.smem > 48 * 1024) PMX_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem));
  // at most one block per SM (route_select_geometry), so the whole grid is resident
  // once the kernels in front of it have drained; the barrier wait is bounded anyway
  return launch_pdl(kern, dim3(g.nblk), dim3(256), g.smem, s, args);
}

int launch_route_select(const void* x, const void* wr, void* scores, void* xp, void* w, int64_t* inv,
                        int64_t* off, int64_t T, int64_t H, int E, int k, int dtype, void* ws,
                        size_t ws_bytes, cudaStream_t s) {
  return launch_route_select_impl(x, wr, scores, xp, w, inv, off, T, H, E, k, dtype, ws, ws_bytes, s, false, NormArgs{});
}

size_t norm_route_select_workspace_bytes(int64_t T, int64_t H, int E, int k, int dtype) {
  RouteSelectGeometry g;
  if (!route_select_geometry(T, H, E, k, dtype, &g, true)) return 0;
  return 64 + (size_t)T * 8;
}

int launch_norm_route_select(const void* x, const void* skip, const void* norm_weight, float eps, const void* wr,
                             void* skip_out, void* scores, void* xp, void* w, int64_t* inv, int64_t* off,
                             int64_t T, int64_t H, int E, int k, int dtype, void* ws, size_t ws_bytes,
                             cudaStream_t s) {
  NormArgs norm{skip, norm_weight, skip_out, eps};
  return launch_route_select_impl(x, wr, scores, xp, w, inv, off, T, H, E, k, dtype, ws, ws_bytes, s, true, norm);
}

// Device address of the built-in scratch on the current device.  Looked up on every
// call (a host-side table lookup once the module is loaded), so that the address is
// never stale after cudaDeviceReset or a change of context on the device.
int select_static_scratch(void** out) {
  void* p = nullptr;
  PMX_CUDA_OK(cudaGetSymbolAddress(&p, g_select_static_scratch));
  if (!p) return fail(PMX_ERR_CUDA, "moe_select_static: cudaGetSymbolAddress returned a null address");
  *out = p;
  return PMX_OK;
}

int launch_select_static(const void* x, const void* scores, void* xp, void* w, int64_t* inv,
                         int64_t* off, int64_t T, int64_t H, int E, int k, int dtype, cudaStream_t s) {
  if (T <= 0 || E <= 0 || k <= 0 || k > E)
    return fail(PMX_ERR_INVALID_ARGUMENT, "moe_select_static: need T > 0 and 0 < k <= E (T=%lld E=%d k=%d)", (long long)T, E, k);
  const size_t need = select_workspace_bytes(T, E, k);
  if (need > (size_t)PMX_MOE_SELECT_STATIC_SCRATCH_BYTES)
    return fail(PMX_ERR_WORKSPACE,
                "moe_select_static: T=%lld E=%d k=%d needs %zu bytes of scratch, the built-in scratch holds %d; "
                "use pmx_moe_select with a workspace of your own",
                (long long)T, E, k, need, (int)PMX_MOE_SELECT_STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  const int st = select_static_scratch(&scratch);
  if (st != PMX_OK) return st;
  // the call prepares what it reads back: ids and per-block counts are
  // overwritten by the routing kernel, the scan's ticket word is cleared by a
  // memset node ahead of the scan; leftovers of earlier calls are never read
  return launch_select(x, scores, xp, w, inv, off, T, H, E, k, dtype, scratch, need, s);
}

}  // namespace pmx
