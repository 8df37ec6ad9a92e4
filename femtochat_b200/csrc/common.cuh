// Shared declarations of libfemto_sm100a: dtype helpers, error plumbing, the GEMM and
// attention entry points used by the model schedule.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/femto.h"

typedef __nv_bfloat16 bf16;

// ---- errors ---------------------------------------------------------------------------------
extern thread_local char g_femto_err[512];
int femto_fail(int code, const char* fmt, ...);
extern long long g_femto_launches;  // host counter of kernel launches issued by the library
#define LAUNCH_COUNT() (++g_femto_launches)

#define CUDA_TRY(expr)                                                                     \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess)                                                                 \
      return femto_fail((int)_e, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),   \
                        __FILE__, __LINE__);                                               \
  } while (0)
#define FEMTO_TRY(expr)        \
  do {                         \
    int _r = (expr);           \
    if (_r != 0) return _r;    \
  } while (0)
#define KERNEL_CHECK()                                                                      \
  do {                                                                                      \
    LAUNCH_COUNT();                                                                         \
    cudaError_t _e = cudaGetLastError();                                                    \
    if (_e != cudaSuccess)                                                                  \
      return femto_fail((int)_e, "kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e), \
                        __FILE__, __LINE__);                                                \
  } while (0)

// Device status word bits (0 = ok).
#define ST_BAD_TOKEN 1u      // token / target / position out of range (clamped, flagged)
#define ST_WAIT_TIMEOUT 2u   // a bounded mbarrier wait ran out
#define ST_NONFINITE 4u

// ---- dtype helpers ----------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }
// Round through the storage type (what the reference's eltype(x).(…) casts do).
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f<T>(from_f<T>(v)); }

template <typename T> struct VecN;  // elements per 16-byte vector
template <> struct VecN<float> { static constexpr int n = 4; };
template <> struct VecN<bf16> { static constexpr int n = 8; };

template <typename T, int V> __device__ __forceinline__ void load_vec(const T* p, float (&f)[V]) {
  if constexpr (V == 1) {
    f[0] = to_f<T>(p[0]);
  } else if constexpr (sizeof(T) == 4) {
    float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  } else {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const bf16* h = reinterpret_cast<const bf16*>(&v);
#pragma unroll
    for (int i = 0; i < 8; i++) f[i] = __bfloat162float(h[i]);
  }
}
template <typename T, int V> __device__ __forceinline__ void store_vec(T* p, const float (&f)[V]) {
  if constexpr (V == 1) {
    p[0] = from_f<T>(f[0]);
  } else if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  } else {
    uint4 v;
    bf16* h = reinterpret_cast<bf16*>(&v);
#pragma unroll
    for (int i = 0; i < 8; i++) h[i] = __float2bfloat16_rn(f[i]);
    *reinterpret_cast<uint4*>(p) = v;
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Per-device one-time set-up (function attributes, device properties): a process may drive several GPUs, and
// cudaFuncSetAttribute / device attributes belong to the device that is current when they are called.
struct PerDevice {
  static constexpr int MAX = 64;
  bool done[MAX] = {};
  int value[MAX] = {};
  // index of the current device, or -1 when it cannot be tracked (then the caller repeats the set-up every time)
  static int current() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX) return -1;
    return dev;
  }
};
// Programmatic dependent launch, primary side: lets a dependent kernel that was launched with the programmatic
// stream-serialisation attribute (the tensor-core GEMM) be scheduled and run its set-up (barriers, tensor memory,
// descriptor prefetch) while this kernel is still running.  The dependent still waits for this kernel's completion
// and memory flush before its first global access (griddepcontrol.wait), so calling this first thing is safe; it
// has no effect when the next kernel is an ordinary launch.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif
int device_sm_count();   // multiprocessors of the current device (cached per device)

static inline int cdiv(long long a, long long b) { return (int)((a + b - 1) / b); }
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- GEMM -------------------------------------------------------------------------------------
// C[M][N] = epilogue(A[M][K] · B[K][N]).  A is stored [M][lda] (K contiguous) when a_kmajor, else
// [K][lda] (M contiguous).  B is stored [N][ldb] (K contiguous) when b_kmajor, else [K][ldb]
// (N contiguous).  C and aux are row-major [M][ld].
enum GemmEpi {
  EPI_STORE = 0,    // C_T = acc
  EPI_RESID = 1,    // C_T = aux_T + acc           (aux may alias C)
  EPI_RELU2 = 2,    // C_T = max(acc,0)^2
  EPI_DRELU2 = 3,   // C_T = acc * 2*sqrt(aux_T)   (aux = relu(u)^2, so 2*sqrt(aux) = 2*max(u,0))
  EPI_AXPBY = 4,    // C_T = alpha*aux_T + beta*acc
  EPI_F32 = 5,      // C_f32 = (beta? C_f32 : 0) + alpha*acc
  EPI_XENT_STATS = 6,   // tensor-core path only: per-row partial (max, sum exp) of softcapped logits; with C set the
                        // logits are also stored there as T
};

struct GemmArgs {
  const void* A = nullptr; const void* B = nullptr; void* C = nullptr; const void* aux = nullptr;
  long long lda = 0, ldb = 0, ldc = 0, ldaux = 0;
  bool a_kmajor = true, b_kmajor = true;
  int M = 0, N = 0, K = 0;
  int epi = EPI_STORE;
  float alpha = 1.f, beta = 0.f;
  int batch = 1;
  long long strideA = 0, strideB = 0, strideC = 0, strideAux = 0;
  // fp32 split output: up to 3 column segments of C go to different destinations (fused QKV dW).
  int nseg = 0; int seg_col0[3] = {0, 0, 0}; int seg_ncol[3] = {0, 0, 0};
  float* seg_ptr[3] = {nullptr, nullptr, nullptr}; long long seg_ld[3] = {0, 0, 0};
  // square symmetric result: tiles that lie entirely below the diagonal are not computed (the caller mirrors
  // the upper triangle afterwards); honoured by the tensor-core kernel, ignored by the SIMT fallback
  bool upper_only = false;
  int ring = 0;   // depth of the operand ring of the tensor-core kernel; 0 = the deepest that fits (fewer stages leave
                  // shared memory free for kernels of another stream to run on the same SMs)
  // cross-entropy statistics epilogue
  const int* targets0 = nullptr;   // [M] 0-based target or -1
  float2* stats = nullptr;         // [M][2 * ntiles_n] partial (max, sumexp)
  float* tz = nullptr;             // [M] softcapped target logit
  int vocab = 0;                   // columns >= vocab are ignored
  // tensor-core path scratch
  void* ws = nullptr; size_t ws_bytes = 0;  // stream-K partials
  unsigned int* status = nullptr;
};

template <typename T> int gemm_simt(const GemmArgs& g, cudaStream_t s);
int gemm_tc_bf16(const GemmArgs& g, cudaStream_t s);       // tcgen05 path (gemm_sm100.cu)
bool gemm_tc_supported(const GemmArgs& g);
template <typename T> int gemm(const GemmArgs& g, cudaStream_t s);  // dispatch

// ---- attention --------------------------------------------------------------------------------
struct AttnArgs {
  void* O = nullptr; float* l = nullptr; float* m = nullptr; float* lse = nullptr;
  const void* Q = nullptr; const void* K = nullptr; const void* V = nullptr;
  // strides in elements between consecutive tokens (rows) of Q/O and of K/V: fused QKV buffers
  long long q_stride = 0, kv_stride = 0, o_stride = 0;
  const void* dO = nullptr; void* dQ = nullptr; void* dK = nullptr; void* dV = nullptr;
  long long do_stride = 0, dq_stride = 0, dkv_stride = 0;
  bool accumulate = false;         // reverse pass: add to dQ / dK / dV instead of overwriting them
  int B = 0, T = 0, H = 0, Hkv = 0, hd = 0, window_left = 0;
  const int* doc_start = nullptr;  // [B][T] or null
  void* ws = nullptr; size_t ws_bytes = 0;
  unsigned int* status = nullptr;
};
template <typename T> int attention_fwd_simt(const AttnArgs& a, cudaStream_t s);
template <typename T> int attention_bwd_simt(const AttnArgs& a, cudaStream_t s);
bool attention_tc_supported(const AttnArgs& a);
int attention_fwd_tc(const AttnArgs& a, cudaStream_t s);
int attention_bwd_tc(const AttnArgs& a, cudaStream_t s);
size_t attention_bwd_tc_ws_bytes(int B, int T, int H, int hd);
template <typename T> int attention_fwd(const AttnArgs& a, cudaStream_t s);
template <typename T> int attention_bwd(const AttnArgs& a, cudaStream_t s);

// ---- embedding scatter ------------------------------------------------------------------------
struct ScatterPlan;   // sorted token order, built once per batch (embed_scatter.cu)
size_t scatter_plan_bytes(int N, int max_cols);
int scatter_plan_create(ScatterPlan** out, int N, int max_cols);
void scatter_plan_destroy(ScatterPlan* p);
int scatter_plan_build(ScatterPlan* p, const int* tokens0, int N, int rows, cudaStream_t s);
template <typename T>
int scatter_rows(ScatterPlan* p, float* table, const T* dy, long long dy_stride, int D, cudaStream_t s);

// ---- deterministic reductions -----------------------------------------------------------------
// out[j] (+)= sum_i partial[i*ncol + j], one block, fixed order.
int reduce_partials(const float* partial, int nrow, int ncol, float* out, const float* scale_dev,
                    float scale, bool accumulate, cudaStream_t s);

// Scratch of the stand-alone kernel-level entry points (femto_attention_bwd, femto_gemm_bf16 with fp32 output,
// femto_xent_fused, femto_newton_schulz, femto_cross_entropy*): one grow-only buffer per device, kept until the
// process exits.  cudaMalloc / cudaFree on every call cost more than the kernels.  Those entry points synchronise
// before returning, so consecutive calls may share it; calls from several host threads at once may not.
int standalone_scratch(size_t bytes, char** out);
// Their status word (bounded waits that ran out, bad token ids): one per device, allocated on first use.
int standalone_status(unsigned int** out);

// ---- lm_head tail ------------------------------------------------------------------------------
// loss rows and (optionally) dX, dW of sum_valid(logsumexp(z) - z[target]), z = 15 tanh(xW/15),
// processed in token chunks; on the tensor-core path a forward-only call writes no logits at all, and a
// call with the reverse pass keeps one chunk of bf16 logits, rewritten in place as d loss/d logit (the
// operand of the two reverse GEMMs).
struct XentArgs {
  const void* x = nullptr; const void* W = nullptr; long long ldw = 0; const int* targets0 = nullptr;
  int N = 0, D = 0, V = 0;
  float scale = 1.f; const float* scale_dev = nullptr;
  bool backward = false; void* dx = nullptr; float* dw = nullptr;
  bool dw_overwrite = false;    // the first chunk's weight gradient overwrites dw instead of adding to it
  int chunk = 0;
  float* logits_f32 = nullptr;  // [chunk][ldw] fp32, SIMT path only
  float2* stats = nullptr; float* tz = nullptr; float* lse_rows = nullptr; float* loss_rows = nullptr;
  void* dlogit = nullptr;       // [chunk][ldw] of T
  void* ws = nullptr; size_t ws_bytes = 0; unsigned int* status = nullptr;
  // Optional second stream for the weight-gradient GEMM of each chunk (with its own split-K workspace, a second
  // dlogit buffer so that the next chunk's logits do not wait for it, and two events + one fork event).
  cudaStream_t side = nullptr; void* ws2 = nullptr; void* dlogit2 = nullptr;
  cudaEvent_t ev_read[2] = {nullptr, nullptr}; cudaEvent_t ev_fork[2] = {nullptr, nullptr};
};
template <typename T> int xent_tail(const XentArgs& x, cudaStream_t s);
bool gemm_profiling();   // per-launch GEMM timing is on: every launch stays on one stream so that the times add up
