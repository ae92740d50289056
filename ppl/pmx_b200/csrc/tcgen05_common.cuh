// Pieces shared by the tcgen05 grouped-GEMM kernels: kernel parameters, PTX wrappers
// (mbarrier, TMA, tensor memory, tcgen05.mma / commit / ld / st), shared-memory and
// instruction descriptors, the bounded barrier wait and the work-item iterator.
// Included inside namespace pmx { namespace { ... } } of each kernel file.
#pragma once

constexpr int kBlockK = 64;      // 16-bit elements per k-block = one 128-byte swizzle row
constexpr int kUmmaK = 16;       // K of one tcgen05.mma with 16-bit operands
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;   // whole tensor memory: 2 accumulator buffers x 256 columns
constexpr int kAccStride = 256;
constexpr int kMaxExperts = 1024;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s
constexpr size_t kStreamKFlagBytes = 1024;                  // room for the per-CTA flags (<= 256 CTAs)

struct Params {
  const int64_t* off;   // [E+1]
  void* y;              // [M, n_out] T   or fp32 partials [split][M][n_out]
  const void* bias;     // [E, N] T or null
  int* status;          // 4 ints: code, role, item, aux
  int M, N, K, E;
  int w_pitch;          // rows between consecutive experts in w (and elements in bias): N unless the
                        // caller passes a window of the feature rows of a wider weight tensor
  int n_out;            // N, or N/2 with SwiGLU
  int tile_tok, tile_feat;
  int feat_tiles;
  int split_k, kb_per_split, kblocks;
  int stages;
  float beta;
  int cta_cap;          // at most this many CTAs take work (the rest of the grid idles)
  int full_rounds;      // shrink the active grid so that every round of tiles is full
  int stream_k;         // 1: the k-blocks of all work items are dealt out evenly over the CTAs
  int* sk_flags;        // [grid] number of epilogue warps that have stored CTA c's partial tile
  float* sk_slots;      // [grid][256 columns][128 lanes] fp32 partial accumulators
  int prefetch;         // weight rows on MMA-M: fetch the weight tiles of the CTA's (guessed) first item
                        // before waiting for the kernel in front
  const int64_t* inv;   // DENSE: invert_permutation [M tokens, k]
  int k;                // DENSE: experts per token
  int balanced;         // weight rows on MMA-M only: every CTA works on a contiguous range of the
                        // feature rows of one (expert, token tile, K slice) panel, or on a run of
                        // whole panels, cut into pieces of at most 128 rows in 8-row units
                        // (feat_tiles is 1 then: a work "item" of the prefix table is a panel)
  int units_per_panel;  // n_out / 8
  unsigned long long* stamps;   // diagnostic: [cta][8] %globaltimer values, or null
  int l2_ahead;         // weight rows on MMA-M: the producer asks for the weight tiles of the k-block this
                        // many rounds in front of the ring to be brought into L2 (0: no prefetch)
};

// tensor maps over the weights with boxes of 64, 32, 16 and 8 rows: a range of feature
// rows that is not a whole 128-row tile is fetched as at most four of these
struct SmallBoxMaps {
  CUtensorMap m[4];
};

// ----------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// adds to the barrier's pending byte count WITHOUT arriving (the phase cannot complete before
// the matching arrive)
__device__ __forceinline__ void mbar_expect_tx_only(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void stamp(unsigned long long* stamps, int word) {
  if (stamps && blockIdx.x < 160) stamps[blockIdx.x * 8 + word] = global_ns();
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// asks for a tile to be brought into L2 (no shared memory, no barrier): the weight stream of a
// thin shard is limited by the bytes a CTA's ring keeps in flight, not by HBM
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* holder, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(holder)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]^T, 16-bit operands, fp32 accumulate
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// mbarrier arrives once all tcgen05.mma issued so far by this thread are done
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 32 lanes x 16 consecutive fp32 columns: thread i gets lane (base lane + i)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
      "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
      "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
      "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
      "r"(__float_as_uint(v[15]))
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ int ld_acquire_gpu_s32(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes,
// stored with the 128-byte swizzle (8-row groups 1024 bytes apart).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3FFF);  // start address / 16
  d |= static_cast<uint64_t>(1) << 16;                // leading byte offset (unused with swizzle)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;        // stride between 8-row groups / 16
  d |= static_cast<uint64_t>(1) << 46;                // descriptor version of sm_100
  d |= static_cast<uint64_t>(2) << 61;                // 128-byte swizzle
  return d;
}

// tcgen05 instruction descriptor: fp32 accumulator, A and B of type T, both K-major
template <typename T>
__device__ __forceinline__ uint32_t make_idesc(int m, int n) {
  const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

constexpr int kMaxStages = 16;
struct Shared {          // control block placed after the ring stages
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile int abort;
  int discard;           // ring stages filled ahead of the dependency wait that turned out not to be
                         // the first item's: the MMA thread hands them back unused
};

// Bounded wait.  Returns false when the CTA is aborting.
__device__ __forceinline__ bool wait_barrier(uint64_t* bar, uint32_t parity, Shared* sh, int* status,
                                             int role, int item) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (sh->abort) return false;
      if (global_ns() - t0 > kWaitLimitNs) {
        sh->abort = 1;
        if (atomicExch(status, 1) != 1) {
          status[1] = role;
          status[2] = item;
          status[3] = static_cast<int>(blockIdx.x);
        }
        return false;
      }
    }
  }
}

struct Item {
  int e, row0, row_end, f0, kb0, kb1, ks;
  int fn;   // feature rows of the item (balanced mode; tile_feat otherwise)
};

// Maps a work-item index to its tile.  `e` carries over between calls (items
// are visited in increasing order).
__device__ __forceinline__ void decode_item(int item, int& e, const int* s_off, const int* s_prefix,
                                            const Params& p, Item& it) {
  while (item >= s_prefix[e + 1]) ++e;
  const int local = item - s_prefix[e];
  const int rows = s_off[e + 1] - s_off[e];
  const int ntt = (rows + p.tile_tok - 1) / p.tile_tok;
  const int tok = local % ntt, fk = local / ntt;
  const int ft = fk / p.split_k;
  it.ks = fk - ft * p.split_k;
  it.e = e;
  it.row0 = s_off[e] + tok * p.tile_tok;
  it.row_end = s_off[e + 1];
  it.f0 = ft * p.tile_feat;
  it.fn = p.tile_feat;
  it.kb0 = it.ks * p.kb_per_split;
  it.kb1 = min(p.kblocks, it.kb0 + p.kb_per_split);
}

// Walks the work of one CTA.  Plain mode: items blockIdx.x, +gridDim.x, ... with
// their (split-K) k range.  Stream-K mode: the CTA owns the contiguous range
// [c*U/G, (c+1)*U/G) of the U = items * kblocks k-block units and meets it as a
// sequence of segments (item, k range); a segment that does not start at k = 0
// is a partial tile that goes to the CTA's slot, a segment that starts at 0 but
// stops early is finished by its owner from the slots of the following CTAs.
struct WorkIter {
  int e;
  int next_item;
  int grid;             // CTAs that take work: blockIdx.x >= grid idles
  int panel_end;        // balanced: one past my last panel (next_item is the current one)
  long long u, u_end, units;
  __device__ __forceinline__ void init(const Params& p, int total_items) {
    e = 0;
    const int cap = min((int)gridDim.x, p.cta_cap);
    grid = cap;
    if (p.balanced) {
      // Every CTA works on a CONTIGUOUS range of feature rows (measured on B200: 3-6 %
      // faster than tiles dealt round-robin).  With at least as many panels (expert,
      // token tile, K slice) as CTAs every CTA takes a contiguous run of whole panels;
      // with fewer, every panel gets its own group of CTAs (grid / panels of them, the
      // first grid % panels panels one more).
      units = p.units_per_panel;
      u = u_end = 0;
      next_item = panel_end = 0;
      const int c = (int)blockIdx.x;
      if (c >= grid || total_items <= 0) return;
      if (total_items >= grid) {
        next_item = (int)((long long)c * total_items / grid);
        panel_end = (int)((long long)(c + 1) * total_items / grid);
        u_end = units;
      } else {
        // n CTAs are available for my panel; they would each get ceil(units / n) units,
        // i.e. `pieces` k-block passes.  Equal passes cost equal time whatever their rows,
        // and rows that are not whole 128-row tiles need several small copies per round
        // (the single producer thread then limits the rate), so the panel goes to as few
        // CTAs as that number of passes allows, each taking whole tiles.
        const int base = grid / total_items, extra = grid % total_items;
        int panel, idx, n;
        if (c < extra * (base + 1)) {
          panel = c / (base + 1); idx = c % (base + 1); n = base + 1;
        } else {
          const int c2 = c - extra * (base + 1);
          panel = extra + c2 / base; idx = c2 % base; n = base;
        }
        const long long tile_units = p.tile_feat / 8;      // 16, or 32 with two 128-row tiles per stage
        const long long share = (units + n - 1) / n;
        const long long pieces = (share + tile_units - 1) / tile_units;
        const long long per_cta = tile_units * pieces;
        next_item = panel;
        panel_end = panel + 1;
        u = idx * per_cta;
        u_end = u + per_cta < units ? u + per_cta : units;
        if (u >= units) { u = u_end = 0; next_item = panel_end = 0; }
      }
      return;
    }
    if (!p.stream_k && p.full_rounds && total_items > 0) {
      // whole tiles per CTA: use the smallest grid that needs no more rounds than
      // `cap` CTAs would, so that every round is full (896 items -> 7 rounds of
      // 128 CTAs instead of 6 rounds of 148 plus a ragged one)
      const int rounds = (total_items + cap - 1) / cap;
      grid = (total_items + rounds - 1) / rounds;
    }
    next_item = (int)blockIdx.x < grid ? (int)blockIdx.x : total_items;
    units = (long long)total_items * p.kblocks;
    if ((int)blockIdx.x < grid) {
      u = (long long)blockIdx.x * units / grid;
      u_end = (long long)(blockIdx.x + 1) * units / grid;
    } else {
      u = u_end = 0;
    }
  }
  __device__ __forceinline__ bool next(const Params& p, int total_items, const int* s_off,
                                       const int* s_prefix, Item& it, int& item) {
    if (p.balanced) {
      if (u >= u_end) {
        if (next_item + 1 >= panel_end) return false;
        ++next_item;            // next whole panel of my run
        u = 0;
        u_end = units;
      }
      if (next_item >= panel_end || u >= u_end) return false;
      const int panel = next_item;
      while (panel >= s_prefix[e + 1]) ++e;
      const int local = panel - s_prefix[e];
      const int rows = s_off[e + 1] - s_off[e];
      const int ntt = (rows + p.tile_tok - 1) / p.tile_tok;
      const int tok = local % ntt;
      it.ks = local / ntt;
      it.e = e;
      it.row0 = s_off[e] + tok * p.tile_tok;
      it.row_end = s_off[e + 1];
      it.kb0 = it.ks * p.kb_per_split;
      it.kb1 = min(p.kblocks, it.kb0 + p.kb_per_split);
      // my units of this panel, a whole tile (16 units of 8 rows, or 32) at a time
      const int seg = (int)(u_end - u);
      const int tile_units = p.tile_feat / 8;
      const int take = seg < tile_units ? seg : tile_units;
      it.f0 = (int)u * 8;
      it.fn = take * 8;
      item = panel;
      u += take;
      return true;
    }
    if (p.stream_k) {
      if (u >= u_end) return false;
      item = (int)(u / p.kblocks);
      decode_item(item, e, s_off, s_prefix, p, it);
      const long long base = (long long)item * p.kblocks;
      it.kb0 = (int)(u - base);
      it.kb1 = (int)((u_end < base + p.kblocks ? u_end : base + p.kblocks) - base);
      u = base + it.kb1;
      return true;
    }
    if (next_item >= total_items) return false;
    item = next_item;
    decode_item(item, e, s_off, s_prefix, p, it);
    next_item += grid;
    return true;
  }
};

template <typename T>
__device__ __forceinline__ void store16(T* dst, const float (&v)[16]) {
  // 16 consecutive outputs: two 16-byte stores
  float a[8], b[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { a[i] = v[i]; b[i] = v[8 + i]; }
  reinterpret_cast<uint4*>(dst)[0] = pack16<T>(a);
  reinterpret_cast<uint4*>(dst)[1] = pack16<T>(b);
}


// ----------------------------------------------------------------------------- host side
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }
  return fn;
}

// 2-D map over a row-major [rows, cols] matrix of 16-bit elements; boxes of
// [box_rows, 64] elements land in shared memory with the 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
             int dtype) {
  PFN_cuTensorMapEncodeTiled_v12000 fn = encode_fn();
  if (!fn) return fail(PMX_ERR_CUDA, "grouped_linear: cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {kBlockK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = dtype == PMX_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(PMX_ERR_CUDA, "grouped_linear: cuTensorMapEncodeTiled failed with code %d (rows=%llu cols=%llu box_rows=%u)", (int)r, (unsigned long long)rows, (unsigned long long)cols, box_rows);
  return PMX_OK;
}

