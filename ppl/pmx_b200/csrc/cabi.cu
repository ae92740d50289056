// extern "C" entry points declared in include/pmx_moe.h: argument checks,
// kernel choice, error text.  No torch types, no allocation, no host sync.
#include <atomic>
#include <mutex>
#include <unordered_set>
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace pmx {

namespace {
thread_local char g_error[512] = "";
std::atomic<long long> g_launches{0};
std::atomic<int> g_pdl{1};
std::atomic<int> g_l2_prefetch{0};
std::atomic<int> g_weight_prefetch{0};
std::mutex g_stamp_mutex;
unsigned long long* g_stamp_buf = nullptr;
int g_stamp_slots = 0, g_stamp_used = 0;
int g_stamp_kernel[256];
}

// Every kernel asks for the largest shared-memory carve-out, also those that need next to
// none: an SM whose L1 / shared-memory split was set for a small kernel cannot take a CTA of
// an expert GEMM (200 KB) until it has drained, so the GEMM CTAs that should start beside
// the CTAs of the kernel in front (programmatic launch) would wait for them to leave --
// seen on B200 as GEMM CTAs entering 8 us late on exactly the SMs the router occupied.
static int prefer_max_shared(const void* kern) {
  static std::mutex m;
  static std::unordered_set<const void*> done;
  std::lock_guard<std::mutex> lock(m);
  if (done.count(kern)) return PMX_OK;
  PMX_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  done.insert(kern);
  return PMX_OK;
}

int launch_pdl(const void* kern, dim3 grid, dim3 block, size_t smem, cudaStream_t s, void** args) {
  {
    const int st = prefer_max_shared(kern);
    if (st != PMX_OK) return st;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl.load(std::memory_order_relaxed) ? 1 : 0;
  PMX_CUDA_OK(cudaLaunchKernelExC(&cfg, kern, args));
  count_launches(1);
  return PMX_OK;
}

unsigned long long* next_stamp_slot(int kernel_id) {
  std::lock_guard<std::mutex> lock(g_stamp_mutex);
  if (!g_stamp_buf || g_stamp_used >= g_stamp_slots) return nullptr;
  g_stamp_kernel[g_stamp_used] = kernel_id;
  return g_stamp_buf + (size_t)(g_stamp_used++) * kStampCtas * kStampWords;
}

int weight_prefetch_enabled() { return g_weight_prefetch.load(std::memory_order_relaxed); }

int default_l2_prefetch() { return g_l2_prefetch.load(std::memory_order_relaxed); }

void count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return status;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return PMX_OK;
  return fail(PMX_ERR_CUDA, "CUDA error %d (%s) from %s", (int)e, cudaGetErrorString(e), what);
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

namespace {

struct LinearChoice {
  bool tc;
  TcPlan plan;
};

int choose_linear(int64_t M, int64_t N, int64_t K, int E, int dtype, int epilogue,
                  const pmx_gemm_plan* user, LinearChoice* c) {
  if (M <= 0 || N <= 0 || K <= 0 || E <= 0)
    return fail(PMX_ERR_INVALID_ARGUMENT, "grouped_linear: M, N, K, E must be positive (M=%lld N=%lld K=%lld E=%d)", (long long)M, (long long)N, (long long)K, E);
  if (dtype != PMX_DTYPE_F16 && dtype != PMX_DTYPE_BF16 && dtype != PMX_DTYPE_F32)
    return fail(PMX_ERR_UNSUPPORTED, "grouped_linear: unknown dtype %d", dtype);
  if (epilogue != PMX_EPILOGUE_NONE && epilogue != PMX_EPILOGUE_SWIGLU)
    return fail(PMX_ERR_INVALID_ARGUMENT, "grouped_linear: unknown epilogue %d", epilogue);
  if (epilogue == PMX_EPILOGUE_SWIGLU && (N & 1))
    return fail(PMX_ERR_INVALID_ARGUMENT, "grouped_linear: SwiGLU needs an even N");
  const int want = user ? user->kernel : PMX_GEMM_AUTO;
  c->tc = false;
  const int64_t pitch = user ? user->w_expert_pitch : 0;
  if (pitch != 0 && (pitch < N || epilogue == PMX_EPILOGUE_SWIGLU || (user->split_k > 1) || user->stream_k == 1))
    return fail(PMX_ERR_INVALID_ARGUMENT, "grouped_linear: w_expert_pitch (%lld) must be at least N (%lld) and cannot be combined with SwiGLU, split-K or stream-K", (long long)pitch, (long long)N);
  if (want == PMX_GEMM_SIMT) return PMX_OK;
  if (want == PMX_GEMM_TC_TOKENS_M_PAIRED) {
    c->tc = plan_gemm_tc_pair(M, N, K, E, dtype, epilogue, user, &c->plan);
  } else {
    c->tc = plan_gemm_tc(M, N, K, E, dtype, epilogue, user, &c->plan);
    // Large experts (prefill): two SMs per 256-token tile.  Measured on B200 for the
    // Mixtral shapes: 1453 against 1334 TFLOP/s (gate/up), 1416 against 1278 (down); with
    // a few hundred rows per expert the larger token tile wastes more than pairing gains.
    if (c->tc && want == PMX_GEMM_AUTO && c->plan.kernel == PMX_GEMM_TC_TOKENS_M && M / E >= 1024) {
      TcPlan paired;
      if (plan_gemm_tc_pair(M, N, K, E, dtype, epilogue, user, &paired)) c->plan = paired;
    }
  }
  if (c->tc) {
    c->plan.w_pitch = (int)pitch;
    if (pitch != 0 && c->plan.split_k > 1) {     // a window of a wider tensor: whole-K tiles only
      pmx_gemm_plan whole = *user;
      whole.split_k = 1;
      return choose_linear(M, N, K, E, dtype, epilogue, &whole, c);
    }
  }
  if (!c->tc && want != PMX_GEMM_AUTO)
    return fail(PMX_ERR_UNSUPPORTED, "grouped_linear: the requested tensor-core plan does not cover this shape/dtype");
  return PMX_OK;
}

}  // namespace
}  // namespace pmx

using namespace pmx;

extern "C" {

int pmx_moe_abi_version(void) { return PMX_MOE_ABI_VERSION; }

const char* pmx_moe_last_error(void) { return g_error; }

long long pmx_moe_kernel_launches(void) { return g_launches.load(std::memory_order_relaxed); }

int pmx_moe_set_programmatic_launch(int on) {
  return g_pdl.exchange(on ? 1 : 0, std::memory_order_relaxed);
}

const char* pmx_moe_status_string(int status) {
  switch (status) {
    case PMX_OK: return "ok";
    case PMX_ERR_INVALID_ARGUMENT: return "invalid argument";
    case PMX_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case PMX_ERR_ALIGNMENT: return "misaligned pointer or pitch";
    case PMX_ERR_WORKSPACE: return "workspace missing or too small";
    case PMX_ERR_CUDA: return "CUDA call failed";
    case PMX_ERR_DEVICE_CHECK: return "device-side self-check failed";
  }
  return "unknown status";
}

size_t pmx_moe_select_workspace_bytes(int64_t T, int32_t E, int32_t k) {
  return select_workspace_bytes(T, E, k);
}

int pmx_moe_select(const void* x, const void* scores, void* x_expand_permute, void* expert_weights,
                   int64_t* invert_permutation, int64_t* expert_offset, int64_t T, int64_t H,
                   int32_t E, int32_t k, int32_t dtype, void* workspace, size_t workspace_bytes,
                   void* stream) {
  return launch_select(x, scores, x_expand_permute, expert_weights, invert_permutation, expert_offset,
                       T, H, E, k, dtype, workspace, workspace_bytes, (cudaStream_t)stream);
}

size_t pmx_moe_route_select_workspace_bytes(int64_t T, int64_t H, int32_t E, int32_t k, int32_t dtype) {
  return route_select_workspace_bytes(T, H, E, k, dtype);
}

int pmx_moe_route_select(const void* x, const void* w_router, void* scores, void* x_expand_permute,
                         void* expert_weights, int64_t* invert_permutation, int64_t* expert_offset,
                         int64_t T, int64_t H, int32_t E, int32_t k, int32_t dtype, void* workspace,
                         size_t workspace_bytes, void* stream) {
  return launch_route_select(x, w_router, scores, x_expand_permute, expert_weights, invert_permutation,
                             expert_offset, T, H, E, k, dtype, workspace, workspace_bytes, (cudaStream_t)stream);
}

int pmx_moe_route_select_check(const void* workspace, void* stream) {
  if (!workspace) return fail(PMX_ERR_INVALID_ARGUMENT, "route_select_check: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  int words[8] = {0};
  PMX_CUDA_OK(cudaMemcpyAsync(words, workspace, sizeof(words), cudaMemcpyDeviceToHost, s));
  PMX_CUDA_OK(cudaStreamSynchronize(s));
  if (words[4] != 0)
    return fail(PMX_ERR_DEVICE_CHECK, "route_select: the grid-wide barrier gave up waiting (code %d, %d blocks had arrived)", words[4], words[0]);
  return PMX_OK;
}

size_t pmx_moe_norm_route_select_workspace_bytes(int64_t T, int64_t H, int32_t E, int32_t k, int32_t dtype) {
  return norm_route_select_workspace_bytes(T, H, E, k, dtype);
}

int pmx_moe_norm_route_select(const void* x, const void* skip, const void* norm_weight, float eps,
                              const void* w_router, void* skip_out, void* scores, void* x_expand_permute,
                              void* expert_weights, int64_t* invert_permutation, int64_t* expert_offset,
                              int64_t T, int64_t H, int32_t E, int32_t k, int32_t dtype, void* workspace,
                              size_t workspace_bytes, void* stream) {
  return launch_norm_route_select(x, skip, norm_weight, eps, w_router, skip_out, scores, x_expand_permute,
                                  expert_weights, invert_permutation, expert_offset, T, H, E, k, dtype,
                                  workspace, workspace_bytes, (cudaStream_t)stream);
}

int pmx_moe_select_static(const void* x, const void* scores, void* x_expand_permute,
                          void* expert_weights, int64_t* invert_permutation, int64_t* expert_offset,
                          int64_t T, int64_t H, int32_t E, int32_t k, int32_t dtype, void* stream) {
  return launch_select_static(x, scores, x_expand_permute, expert_weights, invert_permutation,
                              expert_offset, T, H, E, k, dtype, (cudaStream_t)stream);
}

size_t pmx_moe_grouped_linear_workspace_bytes(int64_t M, int64_t N, int64_t K, int32_t E,
                                              int32_t dtype, int32_t epilogue,
                                              const pmx_gemm_plan* plan) {
  LinearChoice c;
  if (choose_linear(M, N, K, E, dtype, epilogue, plan, &c) != PMX_OK) return 0;
  if (!c.tc || c.plan.kernel == PMX_GEMM_TC_TOKENS_M_PAIRED) return kStatusBytes;
  return gemm_tc_workspace_bytes(M, N, epilogue, c.plan);
}

int pmx_moe_grouped_linear(const void* x, const int64_t* expert_offset, const void* w,
                           const void* bias, void* y, int64_t M, int64_t N, int64_t K, int32_t E,
                           int32_t dtype, int32_t epilogue, float beta, int32_t zero_outside,
                           const pmx_gemm_plan* plan, void* workspace, size_t workspace_bytes,
                           void* stream) {
  if (!x || !w || !y) return fail(PMX_ERR_INVALID_ARGUMENT, "grouped_linear: null pointer");
  if (!expert_offset && E != 1)
    return fail(PMX_ERR_INVALID_ARGUMENT, "grouped_linear: expert_offset may be null only for a single expert (E=%d)", E);
  if (!expert_offset) zero_outside = 0;   // the one expert owns every row
  LinearChoice c;
  int st = choose_linear(M, N, K, E, dtype, epilogue, plan, &c);
  if (st != PMX_OK) return st;
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t n_out = epilogue == PMX_EPILOGUE_SWIGLU ? N / 2 : N;
  if (!c.tc) {
    if (!workspace || workspace_bytes < kStatusBytes)
      return fail(PMX_ERR_WORKSPACE, "grouped_linear: workspace of %zu bytes needed, %zu given", kStatusBytes, workspace_bytes);
    PMX_CUDA_OK(cudaMemsetAsync(workspace, 0, 16, s));
    st = launch_gemm_simt(x, expert_offset, w, bias, y, M, N, K, E, dtype, epilogue, beta,
                          plan ? plan->w_expert_pitch : 0, s);
    if (st != PMX_OK) return st;
    if (zero_outside) return launch_zero_outside(y, expert_offset, M, n_out, E, dtype, s);
    return PMX_OK;
  }
  if (c.plan.kernel == PMX_GEMM_TC_TOKENS_M_PAIRED)
    st = launch_gemm_tc_pair(x, expert_offset, w, bias, y, M, N, K, E, dtype, epilogue, beta, c.plan,
                             workspace, workspace_bytes, s);
  else
    st = launch_gemm_tc(x, expert_offset, w, bias, y, M, N, K, E, dtype, epilogue, beta, c.plan,
                        workspace, workspace_bytes, s);
  if (st != PMX_OK) return st;
  // with split-K the final sum already writes zeros to rows no expert owns
  if (zero_outside && c.plan.split_k == 1) return launch_zero_outside(y, expert_offset, M, n_out, E, dtype, s);
  return PMX_OK;
}

int pmx_moe_dense_gate_up_covers(int64_t T, int64_t N, int64_t K, int32_t E, int32_t k, int32_t dtype) {
  return dense_gate_up_covers(T, N, K, E, k, dtype) ? 1 : 0;
}

int pmx_moe_dense_gate_up(const void* x, const int64_t* invert_permutation, const int64_t* expert_offset,
                          const void* w, const void* bias, void* h, int64_t T, int64_t N, int64_t K, int32_t E,
                          int32_t k, int32_t dtype, float beta, void* workspace, size_t workspace_bytes,
                          void* stream) {
  return launch_gemm_tc_dense(x, invert_permutation, expert_offset, w, bias, h, T, N, K, E, k, dtype, beta,
                              workspace, workspace_bytes, (cudaStream_t)stream);
}

int pmx_moe_set_stamp_buffer(void* buffer, size_t bytes) {
  std::lock_guard<std::mutex> lock(g_stamp_mutex);
  const size_t slot = (size_t)kStampCtas * kStampWords * sizeof(unsigned long long);
  g_stamp_buf = reinterpret_cast<unsigned long long*>(buffer);
  g_stamp_slots = buffer ? (int)(bytes / slot < 256 ? bytes / slot : 256) : 0;
  g_stamp_used = 0;
  return g_stamp_slots;
}

int pmx_moe_stamp_slots(int32_t* kernel_ids, int32_t max_ids) {
  std::lock_guard<std::mutex> lock(g_stamp_mutex);
  for (int i = 0; i < g_stamp_used && i < max_ids; ++i) kernel_ids[i] = g_stamp_kernel[i];
  return g_stamp_used;
}

int pmx_moe_set_weight_prefetch(int on) {
  return g_weight_prefetch.exchange(on ? 1 : 0, std::memory_order_relaxed);
}

int pmx_moe_set_l2_prefetch(int32_t kblocks) {
  return g_l2_prefetch.exchange(kblocks < 0 ? 0 : (kblocks > 64 ? 64 : kblocks), std::memory_order_relaxed);
}

int pmx_moe_dense_mlp_set_rows(int32_t rows) { return dense_mlp_set_rows(rows); }

int pmx_moe_dense_mlp_covers(int64_t T, int64_t N, int64_t H, int32_t E, int32_t k, int32_t dtype) {
  return dense_mlp_covers(T, N, H, E, k, dtype) ? 1 : 0;
}

size_t pmx_moe_dense_mlp_workspace_bytes(int32_t E) { return dense_mlp_workspace_bytes(E); }

int pmx_moe_dense_mlp(const void* x, const int64_t* invert_permutation, const int64_t* expert_offset, const void* wu,
                      const void* w2, void* h, void* y, int64_t T, int64_t N, int64_t H, int32_t E, int32_t k,
                      int32_t dtype, float beta, void* workspace, size_t workspace_bytes, void* stream) {
  return launch_dense_mlp(x, invert_permutation, expert_offset, wu, w2, h, y, T, N, H, E, k, dtype, beta, workspace,
                          workspace_bytes, (cudaStream_t)stream);
}

int pmx_moe_dense_mlp_check(void* workspace, int32_t E, int32_t out[4], void* stream) {
  if (!workspace || !out || E < 1) return fail(PMX_ERR_INVALID_ARGUMENT, "dense_mlp_check: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  PMX_CUDA_OK(cudaMemcpyAsync(out, workspace, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  PMX_CUDA_OK(cudaStreamSynchronize(s));
  if (out[0] != 0) {
    // a launch that gave up may have left its counters behind: put the workspace back to zero
    PMX_CUDA_OK(cudaMemsetAsync(workspace, 0, dense_mlp_workspace_bytes(E), s));
    PMX_CUDA_OK(cudaStreamSynchronize(s));
    return fail(PMX_ERR_DEVICE_CHECK, "dense_mlp: a bounded wait ran out (role %d, work item %d, CTA %d)", out[1], out[2], out[3]);
  }
  return PMX_OK;
}

int pmx_moe_grouped_linear_check(const void* workspace, int32_t out[4], void* stream) {
  if (!workspace || !out) return fail(PMX_ERR_INVALID_ARGUMENT, "grouped_linear_check: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  PMX_CUDA_OK(cudaMemcpyAsync(out, workspace, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  PMX_CUDA_OK(cudaStreamSynchronize(s));
  if (out[0] != 0)
    return fail(PMX_ERR_DEVICE_CHECK, "grouped_linear: a bounded wait ran out (role %d, work item %d, CTA %d)", out[1], out[2], out[3]);
  return PMX_OK;
}

int pmx_swiglu(const void* x, void* y, int64_t M, int64_t D, float beta, int32_t dtype, void* stream) {
  return launch_swiglu(x, y, M, D, beta, dtype, (cudaStream_t)stream);
}

int pmx_silu(const void* x, const void* gate, void* y, int64_t n, int32_t dtype, void* stream) {
  return launch_silu(x, gate, y, n, dtype, (cudaStream_t)stream);
}

int pmx_skip_rms_norm(const void* x, const void* skip, const void* weight, void* y, void* skip_out,
                      int64_t M, int64_t H, float eps, int32_t dtype, void* stream) {
  return launch_skip_rms_norm(x, skip, weight, y, skip_out, M, H, eps, dtype, (cudaStream_t)stream);
}

int pmx_moe_reduce(const void* y, const void* expert_weights, const int64_t* invert_permutation,
                   void* out, int64_t T, int32_t k, int64_t N, int32_t dtype, void* stream) {
  return launch_reduce(y, expert_weights, invert_permutation, out, T, k, N, dtype, (cudaStream_t)stream);
}

int pmx_decode_cache_attention_set_kernel(int32_t kernel) { return decode_attention_set_variant(kernel); }

size_t pmx_decode_cache_attention_workspace_bytes(int64_t B, int32_t num_heads, int32_t num_kv_heads,
                                                  int32_t head_dim, int64_t max_kvlen) {
  return decode_attention_workspace_bytes(B, num_heads, num_kv_heads, head_dim, max_kvlen);
}

int pmx_decode_cache_attention(const void* query, const void* current_key, const void* current_value, void* cache,
                               const int64_t* cachestarts, const int64_t* start_pos, void* out, int64_t B,
                               int32_t num_heads, int32_t num_kv_heads, int32_t head_dim, int64_t layer_offset,
                               int64_t row_stride, int64_t kv_stride, int64_t head_stride, int64_t max_kvlen,
                               int32_t dtype, void* workspace, size_t workspace_bytes, void* stream) {
  return launch_decode_attention(query, current_key, current_value, cache, cachestarts, start_pos, out, B, num_heads,
                                 num_kv_heads, head_dim, layer_offset, row_stride, kv_stride, head_stride, max_kvlen,
                                 dtype, workspace, workspace_bytes, (cudaStream_t)stream);
}

size_t pmx_moe_reduce_allreduce_buffer_bytes(int64_t T, int64_t N, int32_t dtype) {
  if (T <= 0 || N <= 0) return 0;
  return reduce_allreduce_buffer_bytes(T, N, dtype);
}

int pmx_moe_reduce_allreduce(const void* y, const void* expert_weights, const int64_t* invert_permutation,
                             void* out, int64_t T, int32_t k, int64_t N, int32_t dtype,
                             void* const* peer_buffers, int32_t rank, int32_t world,
                             size_t buffer_bytes, int32_t algorithm, int32_t flags, int64_t wait_limit_ns,
                             void* stream) {
  return launch_reduce_allreduce(y, expert_weights, invert_permutation, out, T, k, N, dtype, peer_buffers,
                                 rank, world, buffer_bytes, algorithm, flags, wait_limit_ns, (cudaStream_t)stream);
}

int pmx_moe_reduce_allreduce_emulated(const void* const* y, const void* const* expert_weights,
                                      const int64_t* const* invert_permutation, void* const* out, int64_t T,
                                      int32_t k, int64_t N, int32_t dtype, void* const* buffers, int32_t world,
                                      size_t buffer_bytes, int32_t algorithm, int64_t wait_limit_ns, void* stream) {
  return launch_reduce_allreduce_emulated(y, expert_weights, invert_permutation, out, T, k, N, dtype, buffers,
                                          world, buffer_bytes, algorithm, wait_limit_ns, (cudaStream_t)stream);
}

int pmx_moe_reduce_allreduce_check(void* my_buffer, int32_t out[4], void* stream) {
  if (!my_buffer || !out) return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce_allreduce_check: null pointer");
  return reduce_allreduce_check(my_buffer, out, (cudaStream_t)stream);
}

int pmx_moe_reduce_allreduce_phases(const void* my_buffer, uint64_t out[8], void* stream) {
  if (!my_buffer || !out) return fail(PMX_ERR_INVALID_ARGUMENT, "moe_reduce_allreduce_phases: null pointer");
  return reduce_allreduce_phases(my_buffer, reinterpret_cast<unsigned long long*>(out), (cudaStream_t)stream);
}

}  // extern "C"
