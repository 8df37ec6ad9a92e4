// lm_head tail: softcap + cross-entropy + its reverse (src/gpt.jl:165-170,172-194;
// src/kernels.jl:16-28; ext/FemtoChatEnzymeExt.jl:175-189), in token chunks.
// Tensor-core path (bf16, aligned): pass 1 is a GEMM whose epilogue reduces each row to (max, sum exp)
// partials and the target logit and, for the reverse pass, stores the chunk's logits in bf16; a
// streaming pass rewrites that chunk in place as d loss/d logit, which feeds the dX and dW GEMMs
// (forward-only calls store nothing).  fp32 / unaligned shapes materialise an fp32 logits chunk.
#include <algorithm>

#include "common.cuh"
#include "streaming.cuh"

template <typename T> int xent_tail(const XentArgs& x, cudaStream_t s) {
  const int N = x.N, d = x.D, V = x.V;
  const long long ld = x.ldw;
  const bool two = x.backward && x.side && x.ws2 && x.dlogit2 && x.ev_read[0] && x.ev_read[1] && x.ev_fork[0] && x.ev_fork[1];
  bool armed[2] = {false, false};
  int ci = 0;
  for (int c0 = 0; c0 < N; c0 += x.chunk, ci++) {
    const int cn = std::min(x.chunk, N - c0);
    const T* xc = (const T*)x.x + (size_t)c0 * d;
    void* dlogit = (two && (ci & 1)) ? x.dlogit2 : x.dlogit;
    // the chunk two back handed this buffer to the side stream's weight-gradient GEMM: wait for that reader
    if (two && armed[ci & 1]) { CUDA_TRY(cudaStreamWaitEvent(s, x.ev_read[ci & 1], 0)); armed[ci & 1] = false; }
    GemmArgs g;
    g.ws = x.ws; g.ws_bytes = x.ws_bytes; g.status = x.status; g.ring = two ? 5 : 0;
    g.A = xc; g.lda = d; g.B = x.W; g.ldb = ld; g.b_kmajor = false; g.M = cn; g.N = V; g.K = d;
    g.targets0 = x.targets0 + c0; g.vocab = V;
    g.epi = EPI_XENT_STATS; g.stats = x.stats; g.tz = x.tz + c0;
    // reverse pass: the statistics GEMM also keeps the chunk's logits in bf16 (as the reference materialises
    // them) and a streaming pass turns them into d loss/d logit in place
    if (x.backward) { g.C = dlogit; g.ldc = ld; }
    const bool tc = sizeof(T) == 2 && gemm_tc_supported(g);
    if (tc) {
      FEMTO_TRY(gemm_tc_bf16(g, s));
      FEMTO_TRY(xent_finalize(x.stats, 2 * ((V + 255) / 256), x.tz + c0, x.targets0 + c0, cn, x.lse_rows + c0,
                              x.loss_rows + c0, s));
      if (x.backward)
        FEMTO_TRY(xent_dlogit_inplace(dlogit, ld, x.lse_rows + c0, x.targets0 + c0, cn, V, x.scale, x.scale_dev, s));
    } else {
      if (!x.logits_f32) return femto_fail(FEMTO_ERR_UNSUPPORTED, "lm_head tail: no fp32 logits workspace for this shape");
      g.epi = EPI_F32; g.beta = 0.f; g.C = x.logits_f32; g.ldc = ld;
      FEMTO_TRY(gemm<T>(g, s));
      FEMTO_TRY(Stream<T>::xent_rows(x.logits_f32, ld, x.targets0 + c0, cn, V, x.scale, x.scale_dev, (T*)dlogit, ld,
                                     x.loss_rows + c0, s));
    }
    if (x.backward) {
      cudaStream_t sw = s;
      if (two) {   // the side stream may start once d loss/d logit of this chunk is complete
        CUDA_TRY(cudaEventRecord(x.ev_fork[ci & 1], s));
        CUDA_TRY(cudaStreamWaitEvent(x.side, x.ev_fork[ci & 1], 0));
        sw = x.side;
      }
      GemmArgs gx;  // dx[cn][d] = dlogit[cn][V] * W[d][V]^T
      gx.ws = x.ws; gx.ws_bytes = x.ws_bytes; gx.status = x.status; gx.ring = two ? 5 : 0;
      gx.A = dlogit; gx.lda = ld; gx.B = x.W; gx.ldb = ld; gx.b_kmajor = true; gx.C = (T*)x.dx + (size_t)c0 * d;
      gx.ldc = d; gx.M = cn; gx.N = d; gx.K = V;
      FEMTO_TRY(gemm<T>(gx, s));
      GemmArgs gw;  // dW[d][ld] += x[cn][d]^T * dlogit[cn][V]   (the chunks' sums stay in order: one stream)
      gw.ws = two ? x.ws2 : x.ws; gw.ws_bytes = x.ws_bytes; gw.status = x.status; gw.ring = two ? 5 : 0;
      gw.A = xc; gw.lda = d; gw.a_kmajor = false; gw.B = dlogit; gw.ldb = ld; gw.b_kmajor = false;
      gw.C = x.dw; gw.ldc = ld; gw.M = d; gw.N = V; gw.K = cn; gw.epi = EPI_F32; gw.beta = (x.dw_overwrite && c0 == 0) ? 0.f : 1.f;
      FEMTO_TRY(gemm<T>(gw, sw));
      if (two) { CUDA_TRY(cudaEventRecord(x.ev_read[ci & 1], x.side)); armed[ci & 1] = true; }
    }
  }
  return 0;
}
template int xent_tail<float>(const XentArgs&, cudaStream_t);
template int xent_tail<bf16>(const XentArgs&, cudaStream_t);

extern "C" int32_t femto_xent_fused(int32_t dtype, const void* x, const void* W, int64_t ldw, const int32_t* targets0,
                                    int32_t N, int32_t D, int32_t V, float scale, void* dx, float* dw, float* loss_out,
                                    int32_t* n_valid_out, void* stream) {
  if (!x || !W || !targets0 || !loss_out || N <= 0 || D <= 0 || V <= 0 || ldw < V)
    return femto_fail(FEMTO_ERR_ARG, "bad argument");
  if ((dx == nullptr) != (dw == nullptr)) return femto_fail(FEMTO_ERR_ARG, "dx and dw must both be given or both NULL");
  cudaStream_t s = (cudaStream_t)stream;
  const size_t es = dtype == FEMTO_BF16 ? 2 : 4;
  const int chunk = std::min(N, 8192);
  auto al = [](size_t b) { return (b + 255) & ~(size_t)255; };
  const size_t wsb = (size_t)160 << 20;
  bool need_f32 = dtype != FEMTO_BF16;
  if (!need_f32) {  // the fp32 logits chunk is needed whenever the tensor-core GEMM does not take the shape
    GemmArgs g;
    g.A = x; g.lda = D; g.B = W; g.ldb = ldw; g.b_kmajor = false; g.M = chunk; g.N = V; g.K = D;
    g.epi = EPI_XENT_STATS; g.stats = reinterpret_cast<float2*>(1); g.tz = reinterpret_cast<float*>(1); g.targets0 = targets0;
    need_f32 = !gemm_tc_supported(g);
  }
  size_t total = al(need_f32 ? 4 * (size_t)chunk * ldw : 0) + al(sizeof(float2) * (size_t)chunk * (2 * ((V + 255) / 256) + 2)) +
                 3 * al(4 * (size_t)N) + al(es * (size_t)chunk * ldw) + wsb + 1024;
  char* buf = nullptr;
  FEMTO_TRY(standalone_scratch(total, &buf));
  char* p = buf;
  XentArgs a;
  a.x = x; a.W = W; a.ldw = ldw; a.targets0 = targets0; a.N = N; a.D = D; a.V = V; a.scale = scale;
  a.backward = dx != nullptr; a.dx = dx; a.dw = dw; a.chunk = chunk;
  if (need_f32) { a.logits_f32 = (float*)p; p += al(4 * (size_t)chunk * ldw); }
  a.stats = (float2*)p; p += al(sizeof(float2) * (size_t)chunk * (2 * ((V + 255) / 256) + 2));
  a.tz = (float*)p; p += al(4 * (size_t)N);
  a.lse_rows = (float*)p; p += al(4 * (size_t)N);
  a.loss_rows = (float*)p; p += al(4 * (size_t)N);
  a.dlogit = p; p += al(es * (size_t)chunk * ldw);
  a.ws = p; a.ws_bytes = wsb;
  FEMTO_TRY(standalone_status(&a.status));
  int r = dtype == FEMTO_BF16 ? xent_tail<bf16>(a, s) : xent_tail<float>(a, s);
  if (!r) r = sum_rows_to_scalar(a.loss_rows, N, loss_out, targets0, n_valid_out, 0.f, s);
  cudaStreamSynchronize(s);
  if (!r) {
    unsigned int w = 0;
    CUDA_TRY(cudaMemcpy(&w, a.status, sizeof(w), cudaMemcpyDeviceToHost));
    if (w) { cudaMemset(a.status, 0, sizeof(w)); r = femto_fail(FEMTO_ERR_DEVICE_STATUS + (int)w, "device status word %u", w); }
  }
  return r;
}

// ---- cross-entropy on materialised logits (the reference's stand-alone methods) ------------------
namespace {
// One block per row of fp32 logits [N][ldl]: loss = logsumexp(l) - l[target] (src/gpt.jl:175-193), or, in
// reverse, delta += scale (softmax(l) - onehot) for rows with a target (src/kernels.jl:16-28).
// Fixed reduction trees: repeatable.
template <bool REVERSE>
__global__ void __launch_bounds__(256) k_ce_rows(const float* __restrict__ logits, long long ldl,
                                                 const int* __restrict__ tgt0, int V, float* __restrict__ loss_rows,
                                                 float* __restrict__ delta, long long ldd, float scale_host,
                                                 const float* __restrict__ scale_rows, const int* __restrict__ n_valid) {
  pdl_trigger();
  __shared__ float red[8];
  __shared__ float bc;
  const long long row = blockIdx.x;
  const float* l = logits + row * ldl;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tg = tgt0[row];
  if (REVERSE && tg < 0) return;   // ignored rows contribute nothing
  float mx = -INFINITY;
  for (int v = threadIdx.x; v < V; v += 256) mx = fmaxf(mx, l[v]);
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  if (threadIdx.x == 0) { float m = red[0]; for (int i = 1; i < 8; i++) m = fmaxf(m, red[i]); bc = m; }
  __syncthreads();
  mx = bc;
  float sum = 0.f;
  for (int v = threadIdx.x; v < V; v += 256) sum += expf(l[v] - mx);
  sum = warp_sum(sum);
  __syncthreads();
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  if (threadIdx.x == 0) { float a = 0.f; for (int i = 0; i < 8; i++) a += red[i]; bc = a; }
  __syncthreads();
  const float norm = bc;
  if (!REVERSE) {
    if (threadIdx.x == 0) loss_rows[row] = tg >= 0 ? mx + logf(norm) - l[tg] : 0.f;
  } else {
    float w = scale_rows ? scale_rows[row] : scale_host;
    if (n_valid) w /= (float)n_valid[0];
    float* d = delta + row * ldd;
    for (int v = threadIdx.x; v < V; v += 256) d[v] += w * (expf(l[v] - mx) / norm - (v == tg ? 1.f : 0.f));
  }
}
__global__ void __launch_bounds__(1024) k_count_valid(const int* tgt0, int n, int* out) {
  pdl_trigger();
  __shared__ int red[32];
  int c = 0;
  for (int i = threadIdx.x; i < n; i += 1024) c += tgt0[i] >= 0 ? 1 : 0;
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) { int a = 0; for (int i = 0; i < 32; i++) a += red[i]; out[0] = a; }
}
}  // namespace

extern "C" int32_t femto_cross_entropy(const float* logits, int64_t ldl, const int32_t* targets0, int32_t N, int32_t V,
                                       int32_t reduction, float* out, int32_t* n_valid_out, void* stream) {
  if (!logits || !targets0 || !out || N <= 0 || V <= 0 || ldl < V) return femto_fail(FEMTO_ERR_ARG, "bad argument");
  if (reduction < 0 || reduction > 2) return femto_fail(FEMTO_ERR_ARG, "reduction must be 0 (sum), 1 (mean) or 2 (none)");
  cudaStream_t s = (cudaStream_t)stream;
  if (reduction == FEMTO_REDUCTION_NONE) {   // out is [N]
    k_ce_rows<false><<<N, 256, 0, s>>>(logits, ldl, targets0, V, out, nullptr, 0, 0.f, nullptr, nullptr);
    KERNEL_CHECK();
    if (n_valid_out) { k_count_valid<<<1, 1024, 0, s>>>(targets0, N, n_valid_out); KERNEL_CHECK(); }
    return 0;
  }
  char* scratch = nullptr;
  FEMTO_TRY(standalone_scratch(sizeof(float) * (size_t)N, &scratch));
  float* rows = reinterpret_cast<float*>(scratch);
  k_ce_rows<false><<<N, 256, 0, s>>>(logits, ldl, targets0, V, rows, nullptr, 0, 0.f, nullptr, nullptr);
  int r = 0;
  { cudaError_t e = cudaGetLastError(); if (e != cudaSuccess) r = femto_fail((int)e, "cross-entropy kernel launch failed: %s", cudaGetErrorString(e)); }
  if (!r) r = sum_rows_to_scalar(rows, N, out, targets0, n_valid_out, reduction == FEMTO_REDUCTION_MEAN ? 1.f : 0.f, s);
  cudaStreamSynchronize(s);
  return r;
}

extern "C" int32_t femto_cross_entropy_gradient(float* delta, int64_t ldd, const float* logits, int64_t ldl,
                                                const int32_t* targets0, int32_t N, int32_t V, int32_t reduction,
                                                float dy, const float* dy_rows, void* stream) {
  if (!delta || !logits || !targets0 || N <= 0 || V <= 0 || ldl < V || ldd < V) return femto_fail(FEMTO_ERR_ARG, "bad argument");
  if (reduction < 0 || reduction > 2) return femto_fail(FEMTO_ERR_ARG, "reduction must be 0 (sum), 1 (mean) or 2 (none)");
  if (reduction == FEMTO_REDUCTION_NONE && !dy_rows) return femto_fail(FEMTO_ERR_ARG, "reduction none needs dy_rows [N]");
  cudaStream_t s = (cudaStream_t)stream;
  int* nv = nullptr;
  if (reduction == FEMTO_REDUCTION_MEAN) {
    char* scratch = nullptr;
    FEMTO_TRY(standalone_scratch(256, &scratch));
    nv = reinterpret_cast<int*>(scratch);
    k_count_valid<<<1, 1024, 0, s>>>(targets0, N, nv);
  }
  k_ce_rows<true><<<N, 256, 0, s>>>(logits, ldl, targets0, V, nullptr, delta, ldd, dy,
                                    reduction == FEMTO_REDUCTION_NONE ? dy_rows : nullptr, nv);
  int r = 0;
  { cudaError_t e = cudaGetLastError(); if (e != cudaSuccess) r = femto_fail((int)e, "cross-entropy gradient launch failed: %s", cudaGetErrorString(e)); }
  if (nv) cudaStreamSynchronize(s);
  return r;
}
