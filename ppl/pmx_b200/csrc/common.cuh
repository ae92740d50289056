// Shared helpers for the MoE kernels: element-type traits, 128-bit vector
// access, error reporting for the C ABI.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <tuple>

#include "../../../include/pmx_moe.h"

namespace pmx {

// ---- error text kept per host thread for pmx_moe_last_error() ---------------
int fail(int status, const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);
int sm_count();  // SMs of the current device (cached per device)
void count_launches(int n);  // adds to the process-wide kernel-launch counter

#define PMX_CUDA_OK(expr)                                 \
  do {                                                    \
    int _s = ::pmx::check_cuda((expr), #expr);            \
    if (_s != PMX_OK) return _s;                          \
  } while (0)

// Launches `kern` with programmatic stream serialisation (programmatic dependent
// launch): the grid may be scheduled while the kernel in front of it on the stream
// is still running, as soon as all of that kernel's CTAs have executed
// pdl_launch_dependents() (or exited).  Kernels launched this way call pdl_wait()
// before their first access to memory another kernel may have written, and write
// nothing to global memory before it.  Counts the launch.  With the process-wide
// switch off (pmx_moe_set_programmatic_launch(0)) it is an ordinary launch.
int launch_pdl(const void* kern, dim3 grid, dim3 block, size_t smem, cudaStream_t s, void** args);

// launch_pdl for a kernel given as a function pointer, with its arguments by value
// (converted to the kernel's parameter types).
template <typename... KArgs, typename... Args>
int launch_pdl_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  static_assert(sizeof...(KArgs) == sizeof...(Args), "argument count does not match the kernel");
  std::tuple<KArgs...> vals(static_cast<KArgs>(args)...);
  void* ptrs[sizeof...(KArgs)];
  int i = 0;
  std::apply([&](auto&... v) { ((ptrs[i++] = (void*)&v), ...); }, vals);
  return launch_pdl((const void*)kern, grid, block, smem, s, ptrs);
}

#ifdef __CUDACC__
// Blocks until the grids this one depends on have completed and their memory is
// visible (a no-op in a grid launched without programmatic serialisation).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the dependent grid be scheduled once every CTA of this grid has said so.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// after every kernel launch: count it, then surface a launch error
#define PMX_LAUNCHED()                       \
  do {                                       \
    ::pmx::count_launches(1);                \
    PMX_CUDA_OK(cudaGetLastError());         \
  } while (0)

// ---- element traits ----------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};

// number of elements in one 16-byte vector
template <typename T> constexpr int kVec = 16 / sizeof(T);

// 16 bytes of T as floats and back
template <typename T>
__device__ __forceinline__ void unpack16(const uint4& v, float (&f)[kVec<T>]) {
  const T* p = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int i = 0; i < kVec<T>; ++i) f[i] = Elem<T>::to_f(p[i]);
}
template <typename T>
__device__ __forceinline__ uint4 pack16(const float (&f)[kVec<T>]) {
  uint4 v;
  T* p = reinterpret_cast<T*>(&v);
#pragma unroll
  for (int i = 0; i < kVec<T>; ++i) p[i] = Elem<T>::from_f(f[i]);
  return v;
}

// expert_offset[e]; a null table stands for ONE expert that owns all M rows (a dense linear)
__device__ __forceinline__ long long offset_at(const int64_t* off, int e, long long M) {
  return off ? (long long)off[e] : (e == 0 ? 0ll : M);
}

// 16 bytes of a tensor that never changes while the library runs (weights): read-only path
__device__ __forceinline__ uint4 ld_nc16(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}
// 16 bytes of a tensor that a kernel in front on the stream (or a collective) produced.  Under
// programmatic dependent launch this kernel is resident BEFORE its producers have finished,
// so such data is not read-only for the kernel's lifetime and must not go through the
// non-coherent path (ld.global.nc / __ldg, or a `const __restrict__` parameter, which lets
// the compiler choose it): a line fetched into an SM's L1 by whatever ran there earlier
// would be served stale.  ld.global.cg reads through L2, where the producers' stores land.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  return __ldcg(reinterpret_cast<const uint4*>(p));
}

__device__ __forceinline__ float swiglu_f(float gate, float up, float beta) {
  // up * gate * sigmoid(beta * gate)
  return up * gate / (1.0f + __expf(-beta * gate));
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- kernels' host launchers (one translation unit each) ---------------------
int launch_select(const void* x, const void* scores, void* xp, void* w, int64_t* inv,
                  int64_t* off, int64_t T, int64_t H, int E, int k, int dtype, void* ws,
                  size_t ws_bytes, cudaStream_t s);
size_t select_workspace_bytes(int64_t T, int E, int k);
size_t route_select_workspace_bytes(int64_t T, int64_t H, int E, int k, int dtype);
int launch_route_select(const void* x, const void* wr, void* scores, void* xp, void* w, int64_t* inv,
                        int64_t* off, int64_t T, int64_t H, int E, int k, int dtype, void* ws,
                        size_t ws_bytes, cudaStream_t s);
size_t norm_route_select_workspace_bytes(int64_t T, int64_t H, int E, int k, int dtype);
int launch_norm_route_select(const void* x, const void* skip, const void* norm_weight, float eps, const void* wr,
                             void* skip_out, void* scores, void* xp, void* w, int64_t* inv, int64_t* off,
                             int64_t T, int64_t H, int E, int k, int dtype, void* ws, size_t ws_bytes,
                             cudaStream_t s);
int launch_select_static(const void* x, const void* scores, void* xp, void* w, int64_t* inv,
                         int64_t* off, int64_t T, int64_t H, int E, int k, int dtype, cudaStream_t s);

int launch_swiglu(const void* x, void* y, int64_t M, int64_t D, float beta, int dtype, cudaStream_t s);
int launch_silu(const void* x, const void* gate, void* y, int64_t n, int dtype, cudaStream_t s);
int launch_skip_rms_norm(const void* x, const void* skip, const void* weight, void* y, void* skip_out,
                         int64_t M, int64_t H, float eps, int dtype, cudaStream_t s);
int launch_reduce(const void* y, const void* w, const int64_t* inv, void* out, int64_t T, int k,
                  int64_t N, int dtype, cudaStream_t s);
size_t reduce_allreduce_buffer_bytes(int64_t T, int64_t N, int dtype);
int launch_reduce_allreduce(const void* y, const void* w, const int64_t* inv, void* out, int64_t T,
                            int k, int64_t N, int dtype, void* const* peer_buffers, int rank,
                            int world, size_t buffer_bytes, int algo, int flags, long long wait_limit_ns,
                            cudaStream_t s);
int launch_reduce_allreduce_emulated(const void* const* y, const void* const* w, const int64_t* const* inv,
                                     void* const* out, int64_t T, int k, int64_t N, int dtype,
                                     void* const* buffers, int world, size_t buffer_bytes, int algo,
                                     long long wait_limit_ns, cudaStream_t s);
int reduce_allreduce_check(void* my_buffer, int out[4], cudaStream_t s);
int reduce_allreduce_phases(const void* my_buffer, unsigned long long out[8], cudaStream_t s);
int decode_attention_set_variant(int variant);
size_t decode_attention_workspace_bytes(int64_t B, int Hq, int Hkv, int D, int64_t max_kvlen);
int launch_decode_attention(const void* q, const void* k_cur, const void* v_cur, void* cache,
                            const int64_t* cachestarts, const int64_t* start_pos, void* out, int64_t B, int Hq,
                            int Hkv, int D, int64_t layer_off, int64_t row_stride, int64_t kv_stride,
                            int64_t head_stride, int64_t max_kvlen, int dtype, void* ws, size_t ws_bytes,
                            cudaStream_t s);
int launch_zero_outside(void* y, const int64_t* off, int64_t M, int64_t n_out, int E, int dtype,
                        cudaStream_t s);
int launch_splitk_finish(const float* partial, const int64_t* off, const void* bias, void* y,
                         int64_t M, int64_t n_out, int E, int split, int dtype, bool swiglu,
                         float beta, cudaStream_t s);

int launch_gemm_simt(const void* x, const int64_t* off, const void* w, const void* bias, void* y,
                     int64_t M, int64_t N, int64_t K, int E, int dtype, int epilogue, float beta,
                     int64_t w_pitch, cudaStream_t s);

struct TcPlan {
  int kernel;      // PMX_GEMM_TC_TOKENS_M or PMX_GEMM_TC_WEIGHTS_M
  int tile_feat;   // output features per tile
  int tile_tok;    // token rows per tile
  int split_k;
  int stages;
  int max_ctas;
  int cta_cap;
  int full_rounds;
  int stream_k;
  int balanced;    // weight rows on MMA-M: contiguous whole-tile ranges per CTA, panels not shared
  int w_pitch;     // rows between experts in w (0: N)
  int l2_ahead;    // k-blocks of weight tiles requested into L2 in front of the ring
};
int default_l2_prefetch();
int weight_prefetch_enabled();   // pmx_moe_set_weight_prefetch
// Diagnostic time stamps (pmx_moe_set_stamp_buffer): the next slot of kStampCtas x kStampWords
// %globaltimer values for one launch of an instrumented kernel, or null when switched off.
constexpr int kStampWords = 8;
constexpr int kStampCtas = 160;
unsigned long long* next_stamp_slot(int kernel_id);   // process-wide default for l2_ahead (pmx_moe_set_l2_prefetch)
// Fills `plan` for the tensor-core kernel or returns false when the shape is
// outside what it covers (the caller then uses the CUDA-core kernel).
bool plan_gemm_tc(int64_t M, int64_t N, int64_t K, int E, int dtype, int epilogue,
                  const pmx_gemm_plan* user, TcPlan* plan);
// n_cols: columns of the accumulator the kernel produces (N, or N/2 when SwiGLU
// runs in the kernel's epilogue)
size_t gemm_tc_workspace_bytes(int64_t M, int64_t N, int epilogue, const TcPlan& plan);
int launch_gemm_tc(const void* x, const int64_t* off, const void* w, const void* bias, void* y,
                   int64_t M, int64_t N, int64_t K, int E, int dtype, int epilogue, float beta,
                   const TcPlan& plan, void* ws, size_t ws_bytes, cudaStream_t s);

bool dense_gate_up_covers(int64_t T, int64_t N, int64_t K, int E, int k, int dtype);
int launch_gemm_tc_dense(const void* x, const int64_t* inv, const int64_t* off, const void* w, const void* bias,
                         void* h, int64_t T, int64_t N, int64_t K, int E, int k, int dtype, float beta, void* ws,
                         size_t ws_bytes, cudaStream_t s);

int dense_mlp_set_rows(int rows);
bool dense_mlp_covers(int64_t T, int64_t N, int64_t H, int E, int k, int dtype);
size_t dense_mlp_workspace_bytes(int E);
int launch_dense_mlp(const void* x, const int64_t* inv, const int64_t* off, const void* wu, const void* w2, void* h,
                     void* y, int64_t T, int64_t N, int64_t H, int E, int k, int dtype, float beta, void* ws,
                     size_t ws_bytes, cudaStream_t s);

bool plan_gemm_tc_pair(int64_t M, int64_t N, int64_t K, int E, int dtype, int epilogue,
                       const pmx_gemm_plan* user, TcPlan* plan);
int launch_gemm_tc_pair(const void* x, const int64_t* off, const void* w, const void* bias, void* y,
                        int64_t M, int64_t N, int64_t K, int E, int dtype, int epilogue, float beta,
                        const TcPlan& plan, void* ws, size_t ws_bytes, cudaStream_t s);

constexpr size_t kStatusBytes = 256;  // head of every grouped-linear workspace

}  // namespace pmx
