/*
 * pmx_moe.h -- C ABI of the B200 (sm_100a) implementation of the OPMX
 * mixture-of-experts inference path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*, it is a cudaStream_t / CUstream), launches on that stream
 * and returns without synchronising the host.  Return value: PMX_OK (0) or a
 * negative pmx_status; pmx_moe_last_error() gives the text of the last failure
 * on the calling thread.  Nothing here allocates or frees device memory; the
 * caller provides the outputs and, where stated, a workspace whose size the
 * matching *_workspace_bytes() function returns.  The entry points that take
 * their scratch from the caller keep no state between calls (apart from
 * per-device lookups cached on first use), so they can be called from several
 * host threads and captured in CUDA graphs.
 *
 * Tensors are dense, row-major, innermost dimension contiguous.  "T1" is the
 * activation type selected by `dtype`.  File:line citations name the OPMX
 * reference operator each entry point replaces.
 */
#ifndef PMX_MOE_H_
#define PMX_MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PMX_MOE_ABI_VERSION 3

/* element type of activations and weights */
typedef enum pmx_dtype {
  PMX_DTYPE_F16 = 0,
  PMX_DTYPE_BF16 = 1,
  PMX_DTYPE_F32 = 2
} pmx_dtype;

typedef enum pmx_status {
  PMX_OK = 0,
  PMX_ERR_INVALID_ARGUMENT = -1, /* null pointer, non-positive size, k > E ... */
  PMX_ERR_UNSUPPORTED = -2,      /* shape or dtype outside what the kernels cover */
  PMX_ERR_ALIGNMENT = -3,        /* a pointer or row pitch is not aligned as required */
  PMX_ERR_WORKSPACE = -4,        /* workspace missing or too small */
  PMX_ERR_CUDA = -5,             /* a CUDA runtime / driver call failed */
  PMX_ERR_DEVICE_CHECK = -6      /* a kernel recorded a failed self-check (bounded wait ran out) */
} pmx_status;

/* what the grouped linear applies to the accumulator before storing */
typedef enum pmx_epilogue {
  PMX_EPILOGUE_NONE = 0,  /* Y = X W^T (+ B) */
  PMX_EPILOGUE_SWIGLU = 1 /* W holds [gate rows ; up rows]; Y = up * gate * sigmoid(beta * gate) */
} pmx_epilogue;

/* which grouped-GEMM kernel to run (PMX_GEMM_AUTO picks from shape and dtype) */
typedef enum pmx_gemm_kernel {
  PMX_GEMM_AUTO = 0,
  PMX_GEMM_TC_TOKENS_M = 1,  /* tcgen05: tokens on the MMA M dimension (prefill shape) */
  PMX_GEMM_TC_WEIGHTS_M = 2, /* tcgen05: weight rows on MMA M, tokens on MMA N (decode shape) */
  PMX_GEMM_SIMT = 3,         /* CUDA-core kernel, exact fp32 arithmetic (the only one for fp32) */
  PMX_GEMM_TC_TOKENS_M_PAIRED = 4 /* tcgen05 cta_group::2: two CTAs (SMs) share a 256-token tile and
                                     each loads half of the weight tile (prefill shape) */
} pmx_gemm_kernel;

/* optional tiling override for pmx_moe_grouped_linear; zero fields mean "choose" */
typedef struct pmx_gemm_plan {
  int32_t kernel;       /* pmx_gemm_kernel */
  int32_t tile_feat;    /* output features per tile */
  int32_t tile_tok;     /* token rows per tile */
  int32_t split_k;      /* number of K slices accumulated through the fp32 workspace */
  int32_t stages;       /* shared-memory pipeline depth */
  int32_t max_ctas;     /* cap on the persistent grid (0 = number of SMs) */
  int32_t stream_k;     /* 0 = choose, 1 = deal k-blocks evenly over the CTAs (partial tiles
                           are exchanged through the workspace; needs the SMs to itself, see
                           pmx_moe_grouped_linear), 2 = whole tiles per CTA */
  int32_t cta_cap;      /* at most this many CTAs of the grid take work items (0 = choose) */
  int32_t full_rounds;  /* 0 = choose, 1 = shrink the working grid on the device so that every
                           round of tiles is full, 2 = every CTA up to cta_cap strides over the tiles */
  int32_t balance;      /* PMX_GEMM_TC_WEIGHTS_M only: 0 = choose, 1 = deal the feature rows evenly
                           over the CTAs in units of 8 rows (every SM streams the same number of
                           weight bytes), 2 = whole 128-row tiles */
  int32_t w_expert_pitch; /* 0: w is a dense [E,N,K] tensor.  Otherwise the number of rows between
                           consecutive experts in memory (and of elements between their biases):
                           w points at a window of N feature rows inside a wider [E,pitch,K]
                           weight tensor, e.g. a slice of the hidden columns of the down
                           projection.  Not with SwiGLU, split-K or stream-K. */
  int32_t l2_prefetch;  /* PMX_GEMM_TC_WEIGHTS_M only: the weight tiles of the k-block this many rounds in
                           front of the shared-memory ring are requested into L2 (0 = the process-wide
                           default, none unless pmx_moe_set_l2_prefetch changed it; negative = none) */
} pmx_gemm_plan;

int pmx_moe_abi_version(void);
const char* pmx_moe_last_error(void);
const char* pmx_moe_status_string(int status);
/* Number of kernels this library has launched (or recorded into a CUDA graph
 * under capture) in this process so far; for benchmark accounting. */
long long pmx_moe_kernel_launches(void);
/* Programmatic dependent launch: by default the kernels of this library are
 * launched with programmatic stream serialisation, so that a kernel's set-up (and,
 * for the expert GEMMs, its first weight tiles) overlaps the tail of the kernel in
 * front of it on the stream; every kernel waits for its predecessors before it reads
 * their results or writes anything.  on = 0 switches to ordinary launches for the
 * whole process.  Returns the previous setting. */
int pmx_moe_set_programmatic_launch(int on);
/* L2 prefetch distance of the weight-streaming expert GEMMs (weight rows on MMA-M, the dense
 * gate/up and the one-launch decode kernels), in k-blocks of 64 elements; 0 = no prefetch.
 * A thin shard's weight stream is limited by the bytes the CTAs' shared-memory rings keep
 * in flight (about 18 MB for 112 CTAs); requests into L2 cost no shared memory.  Process-wide;
 * returns the previous value.  Default 0: on B200 the requests compete with the ring's own
 * loads in the TMA unit and every distance measured was slower (8 k-blocks: the 64-token Mixtral
 * decode step 0.68 ms against 0.47 ms, its 1/8 shard 116 against 94 us). */
int pmx_moe_set_l2_prefetch(int32_t kblocks);
/* Weight rows on MMA-M (routed decode GEMMs): whether a CTA requests the weight tiles of its
 * guessed first work item before it waits for the kernel in front (the guess -- every expert
 * owns rows -- is checked after the wait; a wrong guess hands the stages back unused).
 * Off by default: measured on B200 on the 1/8 shard of the Mixtral layer it made the step
 * SLOWER (64 tokens 99.5 against 96.1 us, 8 tokens 93.0 against 88.6 us: the two-step fill of
 * the first stages and the wrong guesses cost more than the early requests gain) and changed
 * nothing at full size.  Process-wide; returns the previous setting. */
int pmx_moe_set_weight_prefetch(int on);
/* Diagnostic: while a device buffer is set, every launch of the router + select kernel and of
 * the weight-streaming expert GEMMs (also when recorded into a CUDA graph) takes the next slot
 * of 160 x 8 uint64 in it and its CTAs store %globaltimer values there: [cta][0] entry,
 * [1] set-up done, [2] first tile arrived, [3] last MMA issued, [4] epilogue free to store
 * (its dependency wait is over), [5] epilogue done, [6] CTA leaves (router: [1] dependency
 * wait over, [2] grid barrier passed).  Returns the number of slots the buffer holds (at
 * most 256); buffer = NULL switches the stamps off.  pmx_moe_stamp_slots: which kernel
 * took each slot so far (1 router + select, 2 grouped GEMM, 3 dense gate/up, 4 both
 * projections in one launch); returns the number of slots taken. */
int pmx_moe_set_stamp_buffer(void* buffer, size_t bytes);
int pmx_moe_stamp_slots(int32_t* kernel_ids, int32_t max_ids);

/*
 * moe_select -- replaces MoeSelect.forward, torch_function/MoeSelect.py:36-64.
 *   x        [T,H]  T1        scores   [T,E] T1
 *   x_expand_permute [T*k,H] T1   rows grouped by expert, stable in slot order t*k+j
 *   expert_weights   [T,k]  T1    softmax over the k kept logits, descending
 *   invert_permutation [T,k] int64  row of x_expand_permute holding slot t*k+j
 *   expert_offset    [E+1]  int64   prefix sum of rows per expert
 * Ranking rule: higher score first, lower expert index among equal scores.
 * Workspace: pmx_moe_select_workspace_bytes(T,E,k) bytes, 16-byte aligned.
 */
size_t pmx_moe_select_workspace_bytes(int64_t T, int32_t E, int32_t k);
int pmx_moe_select(const void* x, const void* scores, void* x_expand_permute,
                   void* expert_weights, int64_t* invert_permutation,
                   int64_t* expert_offset, int64_t T, int64_t H, int32_t E,
                   int32_t k, int32_t dtype, void* workspace,
                   size_t workspace_bytes, void* stream);

/*
 * Router gate + moe_select in one launch, for decode-size batches: replaces
 * Linear.forward (torch_function/Linear.py:24-33, the `gate` call at
 * model_zoo/mixtral/modeling/dynamic_batching/Model.py:188) followed by
 * MoeSelect.forward (torch_function/MoeSelect.py:36-64).
 *   x [T,H] T1, w_router [E,H] T1  ->  scores [T,E] T1 = x . w_router^T (fp32
 *   accumulation, one rounding), then the four outputs of pmx_moe_select computed
 *   from exactly those scores.
 * x_expand_permute may be NULL: the gathered rows are then not written (for callers that
 * feed the un-permuted tokens to pmx_moe_dense_gate_up).
 * Covers 1 <= T <= 1024, E <= 64, k <= 32, H*sizeof(T1) a multiple of 16;
 * pmx_moe_route_select_workspace_bytes returns 0 for other shapes (use a linear
 * and pmx_moe_select then).  The blocks of the launch (at most one per SM) meet at
 * one grid-wide barrier whose two counter words are the first 8 bytes of the
 * workspace: the first 64 bytes of the workspace must be ZERO before the first call
 * that uses it; every call that completes leaves them zero again, so a workspace can
 * be kept and reused without clearing (calls that share a workspace must not overlap
 * on the GPU).  The barrier wait is bounded (1 s); if it runs out the outputs are
 * undefined, pmx_moe_route_select_check reports it and the caller clears the first
 * 64 bytes before the next call.
 */
size_t pmx_moe_route_select_workspace_bytes(int64_t T, int64_t H, int32_t E, int32_t k, int32_t dtype);
int pmx_moe_route_select(const void* x, const void* w_router, void* scores,
                         void* x_expand_permute, void* expert_weights,
                         int64_t* invert_permutation, int64_t* expert_offset,
                         int64_t T, int64_t H, int32_t E, int32_t k, int32_t dtype,
                         void* workspace, size_t workspace_bytes, void* stream);

/*
 * The whole front end of the MoE block in one launch, for decode-size batches:
 * SkipRMSNorm.forward (torch_function/RMSNorm.py:42-56, the `ffn_norm` call at
 * model_zoo/mixtral/modeling/dynamic_batching/Model.py:261), the router gate
 * (Linear.py:24-33, Model.py:188) and MoeSelect.forward (MoeSelect.py:36-64):
 *   s = x (+ skip) -> skip_out (the residual stream; skip and skip_out may be NULL together)
 *   n = T1(float(s) * rsqrt(mean(s^2) + eps)) * norm_weight      (kept on chip)
 *   scores = n . w_router^T, then the four outputs of pmx_moe_select for (n, scores);
 *   x_expand_permute holds rows of n.
 * Same shape limits and workspace contract as pmx_moe_route_select, and additionally the normalised rows of a
 * block's tokens must fit in shared memory (workspace_bytes() returns 0 otherwise).
 */
/* Synchronises `stream`; PMX_ERR_DEVICE_CHECK if the grid barrier of a
 * pmx_moe_route_select / pmx_moe_norm_route_select call on this workspace gave up. */
int pmx_moe_route_select_check(const void* workspace, void* stream);
size_t pmx_moe_norm_route_select_workspace_bytes(int64_t T, int64_t H, int32_t E, int32_t k, int32_t dtype);
int pmx_moe_norm_route_select(const void* x, const void* skip, const void* norm_weight, float eps,
                              const void* w_router, void* skip_out, void* scores,
                              void* x_expand_permute, void* expert_weights,
                              int64_t* invert_permutation, int64_t* expert_offset,
                              int64_t T, int64_t H, int32_t E, int32_t k, int32_t dtype,
                              void* workspace, size_t workspace_bytes, void* stream);

/*
 * moe_select without a workspace argument.  Has no counterpart in the OPMX
 * reference: it exists for hosts that may not allocate device memory around
 * the call -- for example an inference-engine plug-in whose enqueue hook is
 * handed its input and output bindings and nothing else, or a server that gave
 * the whole device to its own arena at start-up and treats any later
 * allocation as a bug.  Same inputs, outputs and results as pmx_moe_select;
 * the ids and per-block counts the kernels need are kept in an array of
 * PMX_MOE_SELECT_STATIC_SCRATCH_BYTES bytes that is part of the library's
 * device image (each GPU that loads the library carries it until the process
 * ends).  The call performs no cudaMalloc / cudaFree and calls no allocating
 * library routine.
 *   - Limit: pmx_moe_select_workspace_bytes(T,E,k) must not exceed
 *     PMX_MOE_SELECT_STATIC_SCRATCH_BYTES (1 MiB: e.g. T*k up to 131072 slots
 *     with 8 experts); larger problems get PMX_ERR_WORKSPACE and a message
 *     naming the size, and should use pmx_moe_select.
 *   - Every call looks up the array's device address for the current device
 *     (cudaGetSymbolAddress, a host-side lookup).  The very first use of the
 *     library on a device may make the CUDA runtime load the library's device
 *     image (which holds the array); make that first call before starting any
 *     stream capture.
 *   - All calls on a device share the one array and it keeps whatever the last
 *     call left there.  Nothing in it needs clearing between calls (every byte
 *     a call reads it has written itself first), but two calls whose kernels
 *     overlap on the GPU -- different streams, or different host threads
 *     without ordering -- race on it.  Keep calls on one stream, or order them.
 */
#define PMX_MOE_SELECT_STATIC_SCRATCH_BYTES (1 << 20)
int pmx_moe_select_static(const void* x, const void* scores,
                          void* x_expand_permute, void* expert_weights,
                          int64_t* invert_permutation, int64_t* expert_offset,
                          int64_t T, int64_t H, int32_t E, int32_t k,
                          int32_t dtype, void* stream);

/*
 * Grouped expert linear -- replaces the per-expert F.linear loops of
 * MoeColumnParallelLinear.forward (torch_function/MoeColumnParallelLinear.py:58-69)
 * and MoeRowParallelLinear.forward (torch_function/MoeRowParallelLinear.py:44-55):
 *   y[r,:] = x[r,:] . w[e]^T (+ bias[e])   for expert_offset[e] <= r < expert_offset[e+1]
 *   x [M,K] T1, w [E,N,K] T1 (K contiguous), bias [E,N] T1 or NULL, expert_offset [E+1] int64
 *   y [M,N] T1, or [M,N/2] T1 with PMX_EPILOGUE_SWIGLU (SwiGLU.forward,
 *   torch_function/SwiGLU.py:15-16, applied to the accumulator: rows [0,N/2) of
 *   w[e] are the gate projection, rows [N/2,N) the up projection).
 * With E == 1, expert_offset may be NULL: the one "expert" then owns all M rows,
 * which makes the call a dense linear y = x . w^T (+ bias) -- Linear.forward
 * (torch_function/Linear.py:24-33), and the local product of
 * ColumnParallelLinear.forward / RowParallelLinear.forward
 * (torch_function/ColumnParallelLinear.py:43, RowParallelLinear.py:41).
 * zero_outside != 0 also writes zeros to rows outside [expert_offset[0],
 * expert_offset[E]) as the reference's zero-initialised output has them.
 * Collectives (all-reduce / all-gather of the reference ops) stay with the caller.
 * plan may be NULL.  Workspace: pmx_moe_grouped_linear_workspace_bytes(...).
 */
size_t pmx_moe_grouped_linear_workspace_bytes(int64_t M, int64_t N, int64_t K,
                                              int32_t E, int32_t dtype,
                                              int32_t epilogue,
                                              const pmx_gemm_plan* plan);
int pmx_moe_grouped_linear(const void* x, const int64_t* expert_offset,
                           const void* w, const void* bias, void* y, int64_t M,
                           int64_t N, int64_t K, int32_t E, int32_t dtype,
                           int32_t epilogue, float beta, int32_t zero_outside,
                           const pmx_gemm_plan* plan, void* workspace,
                           size_t workspace_bytes, void* stream);

/*
 * Gate/up projection with SwiGLU for decode-size batches, computed from the UN-permuted
 * tokens so that it can overlap the routing: replaces MoeColumnParallelLinear.forward
 * (torch_function/MoeColumnParallelLinear.py:58-69) + SwiGLU.forward (SwiGLU.py:15-16) as
 * the Mixtral block calls them (Model.py:198-200), taking x [T,K] instead of the gathered
 * rows of moe_select:
 *   h[r,:] = SwiGLU(x[t,:] . w[e]^T (+ bias[e]))  for every token t and every expert e it was
 *   routed to, r = the row of (t,e) in the expert-sorted order, i.e. the entry of
 *   invert_permutation[t,:] that lies in [expert_offset[e], expert_offset[e+1]).
 * h [T*k, N/2] is exactly what pmx_moe_grouped_linear with PMX_EPILOGUE_SWIGLU writes for
 * the gathered rows.  Every expert's weights are streamed once and multiplied with all T
 * tokens (tensor-core work is free at these sizes), so nothing but the final stores depends
 * on the routing: launched directly behind pmx_moe_route_select / pmx_moe_norm_route_select
 * on the same stream, the weight streaming runs WHILE the router works (programmatic
 * dependent launch) and the epilogue waits for it.  Requirements: x must already be complete
 * when the kernel in front of this one on the stream started (it is read before that kernel
 * finishes); invert_permutation / expert_offset are read only after it has finished.
 * Covers T <= 128, float16 / bfloat16 (pmx_moe_dense_gate_up_covers); every expert's weights
 * are read even if no token chose it, so it pays when (nearly) all experts are active.
 * Workspace: 256 bytes, 16-byte aligned (status words, read by pmx_moe_grouped_linear_check).
 */
int pmx_moe_dense_gate_up_covers(int64_t T, int64_t N, int64_t K, int32_t E, int32_t k, int32_t dtype);
int pmx_moe_dense_gate_up(const void* x, const int64_t* invert_permutation,
                          const int64_t* expert_offset, const void* w, const void* bias, void* h,
                          int64_t T, int64_t N, int64_t K, int32_t E, int32_t k, int32_t dtype,
                          float beta, void* workspace, size_t workspace_bytes, void* stream);

/* The two expert projections of a decode-size batch in ONE launch:
 *   h[r,:] = SwiGLU(x[t,:] . wu[e]^T),   y[r,:] = h[r,:] . w2[e]^T
 * for every token t and every expert e it was routed to (r as for pmx_moe_dense_gate_up):
 * MoeColumnParallelLinear.py:58-69 + SwiGLU.py:15-16 + MoeRowParallelLinear.py:44-55 as
 * called at Model.py:198-205, without the launch boundary between the projections (the w2
 * stream is in flight while the last gate/up tiles finish).  x [T,H], wu [E,N,H] =
 * [gate rows ; up rows], w2 [E,H,N/2], h [T*k,N/2] (an output too), y [T*k,H]; no bias.
 * Same contract towards the routing kernel in front as pmx_moe_dense_gate_up.  Covers
 * T <= 128, float16 / bfloat16, N % 16 == 0, H % 8 == 0.  Workspace
 * (pmx_moe_dense_mlp_workspace_bytes, 16-byte aligned): status words + per-expert
 * counters; it must be zero before the first launch that uses it, every completed launch
 * leaves it zero, and launches that share it must not overlap on the GPU.
 * pmx_moe_dense_mlp_check reads the status back (synchronising) like
 * pmx_moe_grouped_linear_check and, after a failure, clears the workspace. */
/* Tuning switch: gate (= up) rows per work item of the first projection, 64..128 in steps of 8;
 * 0 (default) = chosen per shape so that as many CTAs as possible stream with as deep a ring
 * as fits.  Process-wide; returns the previous value. */
int pmx_moe_dense_mlp_set_rows(int32_t rows);
int pmx_moe_dense_mlp_covers(int64_t T, int64_t N, int64_t H, int32_t E, int32_t k, int32_t dtype);
size_t pmx_moe_dense_mlp_workspace_bytes(int32_t E);
int pmx_moe_dense_mlp(const void* x, const int64_t* invert_permutation,
                      const int64_t* expert_offset, const void* wu, const void* w2, void* h, void* y,
                      int64_t T, int64_t N, int64_t H, int32_t E, int32_t k, int32_t dtype, float beta,
                      void* workspace, size_t workspace_bytes, void* stream);
int pmx_moe_dense_mlp_check(void* workspace, int32_t E, int32_t out[4], void* stream);

/* Reads back (synchronising `stream`) the self-check record a grouped-linear
 * launch left in its workspace: out[0] = 0 if clean, else a code; out[1..3] =
 * where it happened.  Returns PMX_ERR_DEVICE_CHECK if a check failed. */
int pmx_moe_grouped_linear_check(const void* workspace, int32_t out[4], void* stream);

/* swiglu -- SwiGLU.forward, torch_function/SwiGLU.py:15-16.  x [M,D] -> y [M,D/2],
 * y = x[:,D/2:] * x[:,:D/2] * sigmoid(beta * x[:,:D/2]). */
int pmx_swiglu(const void* x, void* y, int64_t M, int64_t D, float beta,
               int32_t dtype, void* stream);

/* silu -- SiLU.forward, torch_function/SiLU.py:18-21.  y = silu(x) (* gate), n elements;
 * gate may be NULL. */
int pmx_silu(const void* x, const void* gate, void* y, int64_t n, int32_t dtype,
             void* stream);

/* rms_norm / skip_rms_norm -- RMSNorm.forward and SkipRMSNorm.forward
 * (torch_function/RMSNorm.py:15-24 and :42-56), the normalisation in front of the MoE
 * block (model_zoo/mixtral/modeling/dynamic_batching/Model.py:261), over the last axis:
 *   s = x (+ skip), rounded to T1 and returned in skip_out when skip is given;
 *   y = T1(float(s) * rsqrt(mean(s^2) + eps)) * weight
 * x, skip, y, skip_out [M,H] T1, weight [H] T1; skip and skip_out may be NULL together. */
int pmx_skip_rms_norm(const void* x, const void* skip, const void* weight, void* y,
                      void* skip_out, int64_t M, int64_t H, float eps, int32_t dtype,
                      void* stream);

/* moe_reduce -- MoeReduce.forward, torch_function/MoeReduce.py:23-25.
 *   y [T*k,N] T1, expert_weights [T,k] T1, invert_permutation [T,k] int64
 *   out[t,:] = sum_j expert_weights[t,j] * y[invert_permutation[t,j],:]   [T,N] T1
 * accumulated in fp32, rounded once. */
int pmx_moe_reduce(const void* y, const void* expert_weights,
                   const int64_t* invert_permutation, void* out, int64_t T,
                   int32_t k, int64_t N, int32_t dtype, void* stream);

/*
 * Decode-step attention over the key/value cache -- replaces, for steps in which every
 * sequence contributes ONE new token, MultiHeadCacheAttention.forward
 * (torch_function/dynamic_batching/MultiHeadCacheAttention.py:104-130), i.e.
 * KeyValueCache.forward (dynamic_batching/KeyValueCache.py:86-138; cache_mode 0, no
 * quantisation) followed by MultiHeadAttention.forward (dynamic_batching/MultiHeadAttention.py:54-108):
 *   for every sequence b: the new key / value [num_kv_heads, head_dim] are stored at cache
 *   row cachestarts[b] + start_pos[b]; out[b,h,:] = softmax(q[b,h] . K^T / sqrt(head_dim)) . V
 *   over the start_pos[b] + 1 cached positions of the key/value head h / (num_heads / num_kv_heads).
 * query, out [B, num_heads, head_dim]; current_key, current_value [B, num_kv_heads, head_dim];
 * cachestarts, start_pos [B] int64 on the device.  The cache element (row, kv, head, d), kv = 0
 * for keys and 1 for values, of the layer in question lives at
 *   cache + layer_offset + row*row_stride + kv*kv_stride + head*head_stride + d   (in elements),
 * which covers the four cache layouts of the reference.  max_kvlen >= start_pos[b] + 1 for all b
 * (it sizes the split of the cached positions over the CTAs).  fp32 arithmetic, one rounding
 * of the result.  float16 / bfloat16, head_dim 64 or 128, at most 8 query heads per kv head.
 * Workspace: pmx_decode_cache_attention_workspace_bytes(...) bytes, 16-byte aligned.
 */
/* Which kernel pmx_decode_cache_attention runs: 0 (default) the tensor-core kernel (mma.sync
 * m16n8k16 on tiles staged in shared memory with cp.async), 1 the CUDA-core kernel (16-byte
 * loads straight into registers).  Process-wide; returns the previous value. */
int pmx_decode_cache_attention_set_kernel(int32_t kernel);
size_t pmx_decode_cache_attention_workspace_bytes(int64_t B, int32_t num_heads, int32_t num_kv_heads,
                                                  int32_t head_dim, int64_t max_kvlen);
int pmx_decode_cache_attention(const void* query, const void* current_key, const void* current_value,
                               void* cache, const int64_t* cachestarts, const int64_t* start_pos,
                               void* out, int64_t B, int32_t num_heads, int32_t num_kv_heads,
                               int32_t head_dim, int64_t layer_offset, int64_t row_stride,
                               int64_t kv_stride, int64_t head_stride, int64_t max_kvlen,
                               int32_t dtype, void* workspace, size_t workspace_bytes, void* stream);

/* how pmx_moe_reduce_allreduce moves the partial results between the ranks */
typedef enum pmx_allreduce_algorithm {
  PMX_ALLREDUCE_AUTO = 0,
  PMX_ALLREDUCE_PULL = 1, /* one hop: every rank publishes a per-CTA flag and reads all peers' buffers */
  PMX_ALLREDUCE_PUSH = 2  /* two hops (reduce at an owner rank, then broadcast) of 8-byte words that
                             carry their own flag; no fence, no separate flag (the default) */
} pmx_allreduce_algorithm;
#define PMX_ALLREDUCE_FLAG_STAMPS 1 /* CTA 0 records %globaltimer at its phase boundaries */

/*
 * moe_reduce fused with the tensor-parallel all-reduce over NVLink peer memory:
 *   out[t,:] = sum over ranks r of  sum_j expert_weights[t,j] * y_r[invert_permutation[t,j],:]
 * i.e. MoeReduce.forward (torch_function/MoeReduce.py:23-25) applied to the
 * all-reduced output of MoeRowParallelLinear.forward
 * (torch_function/MoeRowParallelLinear.py:57-58), with the sum over ranks moved
 * after the weighted combine (same sum, another order; [T,N] crosses NVLink
 * instead of [T*k,N]).  Every rank of the group calls it once per step with its
 * own partial y_r; all ranks must pass identical expert_weights and
 * invert_permutation (the routing is replicated), the same T, algorithm and
 * buffer_bytes.  All ranks receive bit-identical results.
 *   peer_buffers: host array of `world` device pointers, entry r = rank r's
 *   exchange buffer of buffer_bytes >= pmx_moe_reduce_allreduce_buffer_bytes(T_max,N,dtype)
 *   bytes, mapped into this process (CUDA IPC / symmetric memory), zeroed once
 *   before the first call and followed by a barrier of the group.  buffer_bytes
 *   (not T) fixes the layout inside the buffer, so calls with different T <= T_max
 *   may follow each other on the same buffers.
 * Meant for decode-size messages; use NCCL above a few MB.  Waits on peers are
 * bounded by wait_limit_ns (<= 0: one second).  A wait that runs out leaves zeros
 * in the rows it covered and a record that pmx_moe_reduce_allreduce_check reports
 * (and clears); the exchange buffers of all ranks must be zeroed again (and the
 * group synchronised) before the next call.  Call the check at step boundaries.
 */
size_t pmx_moe_reduce_allreduce_buffer_bytes(int64_t T, int64_t N, int32_t dtype);
int pmx_moe_reduce_allreduce(const void* y, const void* expert_weights,
                             const int64_t* invert_permutation, void* out,
                             int64_t T, int32_t k, int64_t N, int32_t dtype,
                             void* const* peer_buffers, int32_t rank,
                             int32_t world, size_t buffer_bytes, int32_t algorithm,
                             int32_t flags, int64_t wait_limit_ns, void* stream);
/* Synchronises `stream`; returns PMX_ERR_DEVICE_CHECK (out = code, peer, epoch, CTA)
 * if a wait ran out since the last check, and clears the record. */
int pmx_moe_reduce_allreduce_check(void* my_buffer, int32_t out[4], void* stream);
/* %globaltimer values CTA 0 recorded in the last call made with PMX_ALLREDUCE_FLAG_STAMPS:
 * out[0] start; PUSH: [1] partials sent, [2] owned sums published, [3] all sums received;
 * PULL: [1] combined, [2] flag published, [3] peers seen, [4] summed.  Synchronises `stream`. */
int pmx_moe_reduce_allreduce_phases(const void* my_buffer, uint64_t out[8], void* stream);
/*
 * The same exchange with all `world` ranks played by ONE cooperative launch on ONE
 * GPU (rank = blockIdx.y), for testing the protocol where only one device is
 * available: y, expert_weights, invert_permutation, out and buffers are host arrays
 * of `world` device pointers, all on the current device.
 */
int pmx_moe_reduce_allreduce_emulated(const void* const* y, const void* const* expert_weights,
                                      const int64_t* const* invert_permutation, void* const* out,
                                      int64_t T, int32_t k, int64_t N, int32_t dtype,
                                      void* const* buffers, int32_t world, size_t buffer_bytes,
                                      int32_t algorithm, int64_t wait_limit_ns, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PMX_MOE_H_ */
