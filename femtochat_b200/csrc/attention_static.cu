// Attention reverse pass for callers that must not allocate device memory.
//
// femto_attention_bwd takes its scratch (the per-row terms D = rowsum(dO * O) and lse * log2(e), two
// floats per (batch, head, query)) from a buffer that it allocates with cudaMalloc on its first call and again
// whenever a larger one is needed.  Some callers cannot do that: a host runtime
// that has handed all device memory to its own pool (XLA-style allocators, a Julia session with a
// capped CUDA.jl pool), or code that runs while allocation is forbidden or would synchronise the
// device.  For them the scratch below is compiled into the library image: every GPU that loads the
// library holds these 8 MiB until the process exits, and the entry point never allocates or frees.
#include "common.cuh"

namespace {

constexpr long long STATIC_SCRATCH_FLOATS = 2ll << 20;  // two floats per row: B*H*T <= 1 048 576 (e.g. 32 x 16 x 2048)
static __device__ __align__(256) float g_attn_bwd_scratch[STATIC_SCRATCH_FLOATS];

// Status word of this entry point (a bounded wait that ran out sets bit 2): like the scratch, part of the library
// image, so that reporting needs no allocation either.
static __device__ unsigned int g_attn_bwd_static_status = 0;

constexpr int MAX_DEVICES = 64;
// Device addresses of the two objects above, per device.  Looked up on the first call on each device; the cache is
// not synchronised between host threads (two first calls at once look the address up twice, harmlessly) and is not
// refreshed after cudaDeviceReset.
float* g_scratch_ptr[MAX_DEVICES] = {nullptr};
unsigned int* g_status_ptr[MAX_DEVICES] = {nullptr};

// The array's name is only a host-side handle: the device address has to be asked for, once per
// device, with that device current.
int scratch_for_current_device(float** out) {
  int dev = -1;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) return femto_fail(FEMTO_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
  if (!g_scratch_ptr[dev]) {
    float* p = nullptr;
    CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_attn_bwd_scratch));
    unsigned int* st = nullptr;
    CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&st), g_attn_bwd_static_status));
    g_status_ptr[dev] = st;
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

// Status word of the allocation-free entry point on the current device (0 before its first call there).
unsigned int static_entry_status_word() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES || !g_status_ptr[dev]) return 0;
  unsigned int w = 0;
  if (cudaMemcpy(&w, g_status_ptr[dev], sizeof(w), cudaMemcpyDeviceToHost) != cudaSuccess) return 0;
  if (w) cudaMemset(g_status_ptr[dev], 0, sizeof(w));   // read and clear
  return w;
}

extern "C" int32_t femto_attention_bwd_static(int32_t dtype, void* dQ, void* dK, void* dV, const void* dO, const void* Q,
                                              const void* K, const void* V, const void* O, const float* lse, int32_t B,
                                              int32_t T, int32_t H, int32_t Hkv, int32_t hd, int32_t window_left,
                                              const int32_t* doc_start, void* stream) {
  if (!dQ || !dK || !dV || !dO || !Q || !K || !V || !O || !lse) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  if (B <= 0 || T <= 0 || H <= 0 || Hkv <= 0 || hd <= 0 || H % Hkv != 0) return femto_fail(FEMTO_ERR_SHAPE, "bad attention shape");
  if (dtype != FEMTO_F32 && dtype != FEMTO_BF16) return femto_fail(FEMTO_ERR_ARG, "dtype must be FEMTO_F32 or FEMTO_BF16");
  const long long need = 2ll * B * H * T;
  if (need > STATIC_SCRATCH_FLOATS)
    return femto_fail(FEMTO_ERR_SHAPE,
                      "femto_attention_bwd_static: B*H*T = %lld exceeds the built-in scratch of %lld rows; "
                      "use femto_attention_bwd, which allocates", need / 2, STATIC_SCRATCH_FLOATS / 2);
  float* scratch = nullptr;
  FEMTO_TRY(scratch_for_current_device(&scratch));
  AttnArgs a;
  a.Q = Q; a.K = K; a.V = V; a.O = const_cast<void*>(O);
  a.q_stride = (long long)H * hd; a.o_stride = a.q_stride; a.kv_stride = (long long)Hkv * hd;
  a.B = B; a.T = T; a.H = H; a.Hkv = Hkv; a.hd = hd;
  a.window_left = window_left < 0 ? T : window_left; a.doc_start = doc_start;
  a.lse = const_cast<float*>(lse); a.dO = dO; a.dQ = dQ; a.dK = dK; a.dV = dV;
  a.do_stride = a.q_stride; a.dq_stride = a.q_stride; a.dkv_stride = a.kv_stride;
  // Every element of the scratch that the kernels read is written first by the same call, so nothing in
  // the shared array needs clearing between calls.
  a.ws = scratch; a.ws_bytes = sizeof(float) * (size_t)STATIC_SCRATCH_FLOATS;
  int dev = -1;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < MAX_DEVICES) a.status = g_status_ptr[dev];
  return dtype == FEMTO_BF16 ? attention_bwd<bf16>(a, (cudaStream_t)stream) : attention_bwd<float>(a, (cudaStream_t)stream);
}
