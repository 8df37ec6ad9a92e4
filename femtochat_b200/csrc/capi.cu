// extern "C" surface of libfemto_sm100a (see include/femto.h for the contract of each entry).
#include <string.h>

#include <vector>

#include "model.cuh"
#include "streaming.cuh"

struct femto_optimizer;
int optimizer_state_sizes(femto_handle* h, long long* out4);
int optimizer_create(femto_handle* h, const femto_optimizer_config* cfg, float* adam_m, float* adam_v, float* muon_m,
                     float* muon_v, femto_optimizer** out);
int optimizer_destroy(femto_optimizer* o);
int optimizer_step(femto_optimizer* o, float* theta, const float* delta, float eta, int has_mu, float mu,
                   int has_lambda, float lambda, float n_tokens, cudaStream_t s);
int optimizer_get_t(femto_optimizer* o, int* t, int cap);
int optimizer_set_t(femto_optimizer* o, const int* t, int count);
int optimizer_set_shard(femto_optimizer* o, int rank, int world);
int optimizer_shard_ranges(femto_optimizer* o, long long* out, int cap);
int optimizer_grad_sync(femto_optimizer* o, float* delta, cudaStream_t s);
femto_handle* optimizer_handle(femto_optimizer* o);
int optimizer_state_ranges(femto_optimizer* o, int which, long long* out, int cap);
int optimizer_gather_state(femto_optimizer* o, cudaStream_t s);
int optimizer_set_exchange(femto_optimizer* o, int mode);
int optimizer_gather_theta(femto_optimizer* o, float* theta, cudaStream_t s);
int adamw_launch(float* theta, const float* delta, float* m, float* v, long long n, float alpha, float b1, float b2,
                 float eps, float lam, int t, float n_tokens, cudaStream_t s);
template <typename T>
int newton_schulz_t(T* S, T* S2, T* A, T* B2, int k, int in, int out, const float* coeffs, int steps, void* ws,
                    size_t ws_bytes, unsigned int* status, cudaStream_t s);

static std::string g_create_err;

int standalone_scratch(size_t bytes, char** out) {
  static char* buf[64] = {nullptr};
  static size_t cap[64] = {0};
  int dev = -1;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return femto_fail(FEMTO_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
  if (cap[dev] < bytes) {
    if (buf[dev]) { cudaDeviceSynchronize(); cudaFree(buf[dev]); buf[dev] = nullptr; cap[dev] = 0; }
    cudaError_t e = cudaMalloc(&buf[dev], bytes);
    if (e != cudaSuccess) return femto_fail(FEMTO_ERR_NOMEM, "cudaMalloc of %zu bytes of scratch failed: %s", bytes, cudaGetErrorString(e));
    cap[dev] = bytes;
  }
  *out = buf[dev];
  return 0;
}

// Status word of the stand-alone kernel-level entry points (they have no handle): one word per device, allocated
// on first use and kept until the process exits.  The entry points that synchronise read it back and report a
// bounded wait that ran out as FEMTO_ERR_DEVICE_STATUS + word; femto_status_word(NULL, ..) reads it for the
// asynchronous ones.
static unsigned int* g_sa_status[64] = {nullptr};
int standalone_status(unsigned int** out) {
  int dev = -1;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return femto_fail(FEMTO_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
  if (!g_sa_status[dev]) {
    CUDA_TRY(cudaMalloc(&g_sa_status[dev], 256));
    CUDA_TRY(cudaMemset(g_sa_status[dev], 0, 256));
  }
  *out = g_sa_status[dev];
  return 0;
}
// Synchronise the stream and turn a raised status word into an error code (the word is cleared for the next call).
static int standalone_finish(int rc, unsigned int* status, cudaStream_t s) {
  cudaError_t e = cudaStreamSynchronize(s);
  if (rc) return rc;
  if (e != cudaSuccess) return femto_fail((int)e, "stream synchronisation failed: %s", cudaGetErrorString(e));
  if (!status) return 0;
  unsigned int w = 0;
  CUDA_TRY(cudaMemcpy(&w, status, sizeof(w), cudaMemcpyDeviceToHost));
  if (w) {
    CUDA_TRY(cudaMemset(status, 0, sizeof(w)));
    return femto_fail(FEMTO_ERR_DEVICE_STATUS + (int)w, "device status word %u (2 = a bounded wait ran out: results are incomplete)", w);
  }
  return 0;
}
unsigned int static_entry_status_word();   // attention_static.cu: status of the allocation-free entry point

static int require_device() {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return femto_fail(FEMTO_ERR_UNSUPPORTED, "no CUDA device: libfemto_sm100a has no CPU fallback (%s)",
                      e != cudaSuccess ? cudaGetErrorString(e) : "device count 0");
  return 0;
}

// lse[i] = m[i] + log l[i]: the reference saves the row sum and the row max separately (src/kernels.jl:425-433)
__global__ void k_lse_from_lm(const float* __restrict__ l, const float* __restrict__ m, float* __restrict__ lse, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) lse[i] = m[i] + logf(l[i]);
}

// Plain row gather: out[n][:] = table[tokens0[n]][:] (one warp per row, 16-byte accesses when D allows)
template <typename T, int V>
__global__ void __launch_bounds__(256) k_embed_gather(const T* __restrict__ table, const int* __restrict__ tok0,
                                                      T* __restrict__ out, int N, int D, int rows, unsigned int* status) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= N) return;
  int t = tok0[row];
  if (t < 0 || t >= rows) { if (lane == 0 && status) atomicOr(status, ST_BAD_TOKEN); t = min(max(t, 0), rows - 1); }
  const T* src = table + (long long)t * D;
  T* dst = out + row * D;
  for (int c = lane * V; c < D; c += 32 * V) {
    float f[V];
    load_vec<T, V>(src + c, f);
    store_vec<T, V>(dst + c, f);
  }
}

int muon_direction_standalone(int dtype, float* X_out, const float* G, float* mom, float* v, int k, int in, int out,
                              float mu, float b2, float n_tokens, const float* coeffs, int steps, unsigned int* status,
                              cudaStream_t s);

extern "C" {

int32_t femto_version(void) { return 100; }

const char* femto_last_error(femto_handle* h) {
  (void)h;
  return g_femto_err;
}

int64_t femto_nparams(const femto_config* cfg) {
  std::vector<femto_tensor_desc> td;
  long long n = 0;
  int r = layout_describe(cfg, td, &n, nullptr);
  return r ? (int64_t)r : (int64_t)n;
}

int32_t femto_layout(const femto_config* cfg, femto_tensor_desc* out, int32_t capacity) {
  std::vector<femto_tensor_desc> td;
  int r = layout_describe(cfg, td, nullptr, nullptr);
  if (r) return r;
  for (int i = 0; i < (int)td.size() && i < capacity; i++) out[i] = td[i];
  return (int32_t)td.size();
}

int32_t femto_window_sizes(const femto_config* cfg, int32_t* left, int32_t* ve) {
  std::vector<int> l, v;
  int r = layout_windows(cfg, l, v);
  if (r) return r;
  for (int i = 0; i < cfg->n_layer; i++) {
    if (left) left[i] = l[i];
    if (ve) ve[i] = v[i];
  }
  return 0;
}

int32_t femto_nccl_unique_id(void* id) { return id ? dp_unique_id(id) : femto_fail(FEMTO_ERR_ARG, "NULL id"); }

int32_t femto_create(const femto_config* cfg, int32_t rank, int32_t world, const void* nccl_id, femto_handle** out) {
  if (!out) return femto_fail(FEMTO_ERR_ARG, "h_out is NULL");
  *out = nullptr;
  if (world < 1 || rank < 0 || rank >= world) return femto_fail(FEMTO_ERR_ARG, "bad rank/world %d/%d", rank, world);
  femto_handle* h = new femto_handle();
  int r = model_fill(h, cfg);
  if (r) { delete h; return r; }
  r = require_device();
  if (r) { delete h; return r; }
  h->rank = rank; h->world = world;
  r = model_alloc(h);
  if (!r) r = dp_create(&h->dp, rank, world, nccl_id);
  if (r) { model_free(h); delete h; return r; }
  *out = h;
  return 0;
}

int32_t femto_destroy(femto_handle* h) {
  if (!h) return 0;
  cudaDeviceSynchronize();
  dp_destroy(h->dp);
  model_free(h);
  delete h;
  return 0;
}

int32_t femto_refresh_weights(femto_handle* h, const float* theta, void* stream) {
  if (!h || !theta) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  return model_refresh(h, theta, (cudaStream_t)stream);
}

int32_t femto_loss_and_gradient(femto_handle* h, const float* theta, float* delta, const int32_t* tokens,
                                const int32_t* targets, const int32_t* positions, int32_t B, int32_t reduction,
                                int32_t accumulate, float* loss_out, int32_t* n_valid_out, void* stream) {
  if (!h) return femto_fail(FEMTO_ERR_ARG, "NULL handle");
  return model_step(h, theta, delta, tokens, targets, positions, B, reduction, true, accumulate != 0, loss_out,
                    n_valid_out, (cudaStream_t)stream);
}

int32_t femto_forward_loss(femto_handle* h, const float* theta, const int32_t* tokens, const int32_t* targets,
                           const int32_t* positions, int32_t B, int32_t reduction, float* loss_out,
                           int32_t* n_valid_out, void* stream) {
  if (!h) return femto_fail(FEMTO_ERR_ARG, "NULL handle");
  return model_step(h, theta, nullptr, tokens, targets, positions, B, reduction, false, false, loss_out, n_valid_out,
                    (cudaStream_t)stream);
}

int32_t femto_forward_logits(femto_handle* h, const float* theta, const int32_t* tokens, const int32_t* positions,
                             int32_t B, float* logits_out, void* stream) {
  if (!h || !logits_out) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  return model_step(h, theta, nullptr, tokens, nullptr, positions, B, FEMTO_REDUCTION_SUM, false, false, nullptr, nullptr,
                    (cudaStream_t)stream, logits_out);
}

int32_t femto_forward_token_losses(femto_handle* h, const float* theta, const int32_t* tokens, const int32_t* targets,
                                   const int32_t* positions, int32_t B, float* losses_out, int32_t* n_valid_out,
                                   void* stream) {
  if (!h || !losses_out) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  // the scalar path also counts the valid targets; its sum goes to the handle's own loss scalar
  return model_step(h, theta, nullptr, tokens, targets, positions, B, FEMTO_REDUCTION_SUM, false, false, h->loss_dev,
                    n_valid_out ? n_valid_out : h->nvalid_dev, (cudaStream_t)stream, nullptr, losses_out);
}

int32_t femto_loss_and_gradient_host(femto_handle* h, const float* theta, float* delta, const int32_t* h_tokens,
                                     const int32_t* h_targets, const int32_t* h_positions, int32_t B,
                                     int32_t reduction, int32_t accumulate, float* h_loss, int32_t* h_n_valid,
                                     void* stream) {
  if (!h || !h_tokens || !h_targets || !h_loss) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  if (B <= 0 || B > h->maxB) return femto_fail(FEMTO_ERR_SHAPE, "B=%d outside 1..max_batch=%d", B, h->maxB);
  cudaStream_t s = (cudaStream_t)stream;
  const size_t bytes = sizeof(int) * (size_t)B * h->T;
  CUDA_TRY(cudaMemcpyAsync(h->raw_tok, h_tokens, bytes, cudaMemcpyHostToDevice, s));
  CUDA_TRY(cudaMemcpyAsync(h->raw_tgt, h_targets, bytes, cudaMemcpyHostToDevice, s));
  if (h_positions) CUDA_TRY(cudaMemcpyAsync(h->raw_pos, h_positions, bytes, cudaMemcpyHostToDevice, s));
  FEMTO_TRY(model_step(h, theta, delta, h->raw_tok, h->raw_tgt, h_positions ? h->raw_pos : nullptr, B, reduction, true,
                       accumulate != 0, h->loss_dev, h->nvalid_dev, s));
  int nv = 0;
  CUDA_TRY(cudaMemcpyAsync(h_loss, h->loss_dev, sizeof(float), cudaMemcpyDeviceToHost, s));
  CUDA_TRY(cudaMemcpyAsync(&nv, h->nvalid_dev, sizeof(int), cudaMemcpyDeviceToHost, s));
  CUDA_TRY(cudaStreamSynchronize(s));
  if (h_n_valid) *h_n_valid = nv;
  return 0;
}

int32_t femto_grad_sync(femto_handle* h, float* delta, float* loss_inout, int32_t* n_valid_inout, void* stream) {
  if (!h || !delta) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  if (h->world <= 1) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (h->delta_synced) {
    FEMTO_TRY(dp_join(h->dp, s));   // the buckets were queued by the reverse pass
    h->delta_synced = false;
  } else {
    FEMTO_TRY(dp_allreduce_sum_f32(h->dp, delta, h->nparams, s));
  }
  if (loss_inout) FEMTO_TRY(dp_allreduce_sum_f32(h->dp, loss_inout, 1, s));
  if (n_valid_inout) FEMTO_TRY(dp_allreduce_sum_i32(h->dp, n_valid_inout, 1, s));
  return 0;
}

int32_t femto_comm_check(femto_handle* h) {
  if (!h) return femto_fail(FEMTO_ERR_ARG, "NULL handle");
  return dp_async_error(h->dp);
}
int32_t femto_comm_abort(femto_handle* h) {
  if (!h) return femto_fail(FEMTO_ERR_ARG, "NULL handle");
  return dp_abort(h->dp);
}

int32_t femto_set_overlap(femto_handle* h, int32_t enable) {
  if (!h) return femto_fail(FEMTO_ERR_ARG, "NULL handle");
  h->overlap_sync = enable != 0;
  return 0;
}

int32_t femto_optimizer_state_sizes(femto_handle* h, int64_t* out4) {
  if (!h || !out4) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  long long v[4];
  optimizer_state_sizes(h, v);
  for (int i = 0; i < 4; i++) out4[i] = v[i];
  return 0;
}
int32_t femto_optimizer_create(femto_handle* h, const femto_optimizer_config* cfg, float* adam_m, float* adam_v,
                               float* muon_m, float* muon_v, femto_optimizer** out) {
  return optimizer_create(h, cfg, adam_m, adam_v, muon_m, muon_v, out);
}
int32_t femto_optimizer_destroy(femto_optimizer* o) { return optimizer_destroy(o); }
int32_t femto_optimizer_step(femto_optimizer* o, float* theta, const float* delta, float eta, int32_t has_mu, float mu,
                             int32_t has_lambda, float lambda, float n_tokens, void* stream) {
  return optimizer_step(o, theta, delta, eta, has_mu, mu, has_lambda, lambda, n_tokens, (cudaStream_t)stream);
}
int32_t femto_optimizer_set_shard(femto_optimizer* o, int32_t rank, int32_t world) { return optimizer_set_shard(o, rank, world); }
int32_t femto_optimizer_shard_ranges(femto_optimizer* o, int64_t* h_out, int32_t capacity) {
  if (!o || (capacity > 0 && !h_out)) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  static_assert(sizeof(long long) == sizeof(int64_t), "int64_t");
  return optimizer_shard_ranges(o, (long long*)h_out, capacity);
}
int32_t femto_optimizer_state_ranges(femto_optimizer* o, int32_t which, int64_t* h_out, int32_t capacity) {
  if (!o || (capacity > 0 && !h_out)) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  return optimizer_state_ranges(o, which, (long long*)h_out, capacity);
}
int32_t femto_optimizer_gather_state(femto_optimizer* o, void* stream) {
  if (!o) return femto_fail(FEMTO_ERR_ARG, "NULL optimizer");
  return optimizer_gather_state(o, (cudaStream_t)stream);
}
int32_t femto_optimizer_set_exchange(femto_optimizer* o, int32_t mode) { return optimizer_set_exchange(o, mode); }
int32_t femto_optimizer_gather_theta(femto_optimizer* o, float* theta, void* stream) {
  return optimizer_gather_theta(o, theta, (cudaStream_t)stream);
}
int32_t femto_optimizer_grad_sync(femto_optimizer* o, float* delta, float* loss_inout, int32_t* n_valid_inout, void* stream) {
  if (!o || !delta) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  femto_handle* h = optimizer_handle(o);
  if (h->world <= 1) return 0;
  // buckets already summed during the reverse pass (femto_set_overlap) are complete on every rank
  if (h->delta_synced) return femto_grad_sync(h, delta, loss_inout, n_valid_inout, stream);
  cudaStream_t s = (cudaStream_t)stream;
  FEMTO_TRY(optimizer_grad_sync(o, delta, s));
  if (loss_inout) FEMTO_TRY(dp_allreduce_sum_f32(h->dp, loss_inout, 1, s));
  if (n_valid_inout) FEMTO_TRY(dp_allreduce_sum_i32(h->dp, n_valid_inout, 1, s));
  return 0;
}
int32_t femto_optimizer_get_t(femto_optimizer* o, int32_t* t, int32_t cap) {
  if (!o || !t) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  return optimizer_get_t(o, t, cap);
}
int32_t femto_optimizer_set_t(femto_optimizer* o, const int32_t* t, int32_t count) {
  if (!o || !t) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  return optimizer_set_t(o, t, count);
}

static int fill_attn(AttnArgs& a, const void* Q, const void* K, const void* V, void* O, int B, int T, int H, int Hkv,
                     int hd, int window_left, const int* doc_start) {
  if (!Q || !K || !V || !O) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  if (B <= 0 || T <= 0 || H <= 0 || Hkv <= 0 || hd <= 0 || H % Hkv != 0) return femto_fail(FEMTO_ERR_SHAPE, "bad attention shape");
  a.Q = Q; a.K = K; a.V = V; a.O = O; a.q_stride = (long long)H * hd; a.o_stride = a.q_stride;
  a.kv_stride = (long long)Hkv * hd; a.B = B; a.T = T; a.H = H; a.Hkv = Hkv; a.hd = hd;
  a.window_left = window_left < 0 ? T : window_left; a.doc_start = doc_start;
  return 0;
}

int32_t femto_attention_fwd(int32_t dtype, void* O, float* l, float* m, float* lse, const void* Q, const void* K,
                            const void* V, int32_t B, int32_t T, int32_t H, int32_t Hkv, int32_t hd,
                            int32_t window_left, const int32_t* doc_start, void* stream) {
  FEMTO_TRY(require_device());
  AttnArgs a;
  FEMTO_TRY(fill_attn(a, Q, K, V, O, B, T, H, Hkv, hd, window_left, doc_start));
  a.l = l; a.m = m; a.lse = lse;
  FEMTO_TRY(standalone_status(&a.status));
  return dtype == FEMTO_BF16 ? attention_fwd<bf16>(a, (cudaStream_t)stream) : attention_fwd<float>(a, (cudaStream_t)stream);
}

int32_t femto_attention_bwd(int32_t dtype, void* dQ, void* dK, void* dV, const void* dO, const void* Q, const void* K,
                            const void* V, const void* O, const float* lse, const float* l, const float* m, int32_t B,
                            int32_t T, int32_t H, int32_t Hkv, int32_t hd, int32_t window_left, const int32_t* doc_start,
                            int32_t accumulate, void* stream) {
  FEMTO_TRY(require_device());
  if (!dQ || !dK || !dV || !dO) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  if (!lse && (!l || !m)) return femto_fail(FEMTO_ERR_ARG, "pass lse, or both l and m");
  AttnArgs a;
  FEMTO_TRY(fill_attn(a, Q, K, V, const_cast<void*>(O), B, T, H, Hkv, hd, window_left, doc_start));
  a.dO = dO; a.dQ = dQ; a.dK = dK; a.dV = dV; a.accumulate = accumulate != 0;
  a.do_stride = a.q_stride; a.dq_stride = a.q_stride; a.dkv_stride = a.kv_stride;
  const size_t rows = (size_t)B * H * T;
  const size_t need = (std::max(sizeof(float) * rows * 2, attention_bwd_tc_ws_bytes(B, T, H, hd)) + 255) & ~(size_t)255;
  char* ws = nullptr;
  FEMTO_TRY(standalone_scratch(need + sizeof(float) * rows, &ws));
  a.ws = ws; a.ws_bytes = need;
  cudaStream_t s = (cudaStream_t)stream;
  if (lse) {
    a.lse = const_cast<float*>(lse);
  } else {
    float* tmp = reinterpret_cast<float*>(ws + need);
    k_lse_from_lm<<<cdiv((long long)rows, 256), 256, 0, s>>>(l, m, tmp, (long long)rows);
    KERNEL_CHECK();
    a.lse = tmp;
  }
  FEMTO_TRY(standalone_status(&a.status));
  int r = dtype == FEMTO_BF16 ? attention_bwd<bf16>(a, s) : attention_bwd<float>(a, s);
  return standalone_finish(r, a.status, s);
}

int32_t femto_gemm_bf16(const void* A, int32_t a_kmajor, int64_t lda, const void* B, int32_t b_kmajor, int64_t ldb,
                        void* C, int64_t ldc, int32_t M, int32_t N, int32_t K, int32_t batch, int64_t strideA,
                        int64_t strideB, int64_t strideC, int32_t out_f32, int32_t accumulate, void* stream) {
  FEMTO_TRY(require_device());
  if (!A || !B || !C) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  if (accumulate && !out_f32) return femto_fail(FEMTO_ERR_ARG, "accumulate needs out_f32");
  GemmArgs g;
  g.A = A; g.B = B; g.C = C; g.lda = lda; g.ldb = ldb; g.ldc = ldc; g.a_kmajor = a_kmajor != 0; g.b_kmajor = b_kmajor != 0;
  g.M = M; g.N = N; g.K = K; g.batch = batch < 1 ? 1 : batch; g.strideA = strideA; g.strideB = strideB; g.strideC = strideC;
  g.epi = out_f32 ? EPI_F32 : EPI_STORE; g.beta = accumulate ? 1.f : 0.f;
  FEMTO_TRY(standalone_status(&g.status));
  if (!out_f32) return gemm<bf16>(g, (cudaStream_t)stream);  // asynchronous, no scratch
  char* ws = nullptr;  // split-K partials of the fp32 form
  const size_t wsb = (size_t)160 << 20;
  FEMTO_TRY(standalone_scratch(wsb, &ws));
  g.ws = ws; g.ws_bytes = wsb;
  int r = gemm<bf16>(g, (cudaStream_t)stream);
  return standalone_finish(r, g.status, (cudaStream_t)stream);
}

int32_t femto_embedding_gradient(int32_t dtype, float* table, const void* dy, const int32_t* tokens0, int32_t N,
                                 int32_t D, int32_t rows, void* stream) {
  FEMTO_TRY(require_device());
  if (!table || !dy || !tokens0 || N <= 0 || D <= 0 || rows <= 0) return femto_fail(FEMTO_ERR_ARG, "bad argument");
  // the sort / run-length plan's buffers are kept per device and re-created only for a larger problem
  static ScatterPlan* plan[64] = {nullptr};
  static int plan_n[64] = {0}, plan_d[64] = {0};
  int dev = -1;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return femto_fail(FEMTO_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
  if (!plan[dev] || plan_n[dev] < N || plan_d[dev] < D) {
    if (plan[dev]) { cudaDeviceSynchronize(); scatter_plan_destroy(plan[dev]); plan[dev] = nullptr; }
    FEMTO_TRY(scatter_plan_create(&plan[dev], std::max(N, plan_n[dev]), std::max(D, plan_d[dev])));
    plan_n[dev] = std::max(N, plan_n[dev]); plan_d[dev] = std::max(D, plan_d[dev]);
  }
  ScatterPlan* p = plan[dev];
  cudaStream_t s = (cudaStream_t)stream;
  int r = scatter_plan_build(p, tokens0, N, rows, s);
  if (!r) r = dtype == FEMTO_BF16 ? scatter_rows<bf16>(p, table, (const bf16*)dy, D, D, s)
                                  : scatter_rows<float>(p, table, (const float*)dy, D, D, s);
  cudaStreamSynchronize(s);
  return r;
}

int32_t femto_adamw(float* theta, const float* delta, float* m, float* v, int64_t n, float alpha, float beta1,
                    float beta2, float eps, float lambda, int32_t t, float n_tokens, void* stream) {
  FEMTO_TRY(require_device());
  if (!theta || !delta || !m || !v || n <= 0 || t < 1) return femto_fail(FEMTO_ERR_ARG, "bad argument");
  return adamw_launch(theta, delta, m, v, n, alpha, beta1, beta2, eps, lambda, t, n_tokens, (cudaStream_t)stream);
}

int32_t femto_newton_schulz(int32_t dtype, void* X, int32_t k, int32_t rows, int32_t cols, const float* coeffs,
                            int32_t steps, void* stream) {
  FEMTO_TRY(require_device());
  if (!X || !coeffs || k <= 0 || rows <= 0 || cols <= 0 || steps < 0) return femto_fail(FEMTO_ERR_ARG, "bad argument");
  const size_t es = dtype == FEMTO_BF16 ? 2 : 4;
  const size_t per = (size_t)rows * cols, r = std::min(rows, cols);
  const size_t wsb = (size_t)160 << 20;
  char* buf = nullptr;
  auto al = [](size_t b) { return (b + 255) & ~(size_t)255; };
  FEMTO_TRY(standalone_scratch(al(es * per * k) + 2 * al(es * r * r * k) + wsb + 256, &buf));
  void* S2 = buf;
  void* A = buf + al(es * per * k);
  void* B2 = (char*)A + al(es * r * r * k);
  void* ws = (char*)B2 + al(es * r * r * k);
  cudaStream_t s = (cudaStream_t)stream;
  unsigned int* status = nullptr;
  FEMTO_TRY(standalone_status(&status));
  // row-major [rows][cols] == stored [in=rows][out=cols]
  int rc = dtype == FEMTO_BF16
               ? newton_schulz_t<bf16>((bf16*)X, (bf16*)S2, (bf16*)A, (bf16*)B2, k, rows, cols, coeffs, steps, ws, wsb, status, s)
               : newton_schulz_t<float>((float*)X, (float*)S2, (float*)A, (float*)B2, k, rows, cols, coeffs, steps, ws, wsb, status, s);
  return standalone_finish(rc, status, s);
}

int32_t femto_rmsnorm_fwd(int32_t dtype, const void* x, void* y, float* r, int32_t N, int32_t D, float eps, void* stream) {
  FEMTO_TRY(require_device());
  if (!x || !y || !r || N <= 0 || D <= 0) return femto_fail(FEMTO_ERR_ARG, "bad argument");
  if (dtype != FEMTO_F32 && dtype != FEMTO_BF16) return femto_fail(FEMTO_ERR_ARG, "dtype must be FEMTO_F32 or FEMTO_BF16");
  if (!aligned16(x) || !aligned16(y)) return femto_fail(FEMTO_ERR_ALIGN, "x and y must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  return dtype == FEMTO_BF16 ? Stream<bf16>::norm((const bf16*)x, (bf16*)y, r, N, D, eps, s)
                             : Stream<float>::norm((const float*)x, (float*)y, r, N, D, eps, s);
}

int32_t femto_rmsnorm_bwd(int32_t dtype, const void* dy, const void* y, const float* r, void* dx, int32_t N, int32_t D,
                          void* stream) {
  FEMTO_TRY(require_device());
  if (!dy || !y || !r || !dx || N <= 0 || D <= 0) return femto_fail(FEMTO_ERR_ARG, "bad argument");
  if (dtype != FEMTO_F32 && dtype != FEMTO_BF16) return femto_fail(FEMTO_ERR_ARG, "dtype must be FEMTO_F32 or FEMTO_BF16");
  if (!aligned16(dy) || !aligned16(y) || !aligned16(dx)) return femto_fail(FEMTO_ERR_ALIGN, "dy, y and dx must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  return dtype == FEMTO_BF16 ? Stream<bf16>::norm_bwd_resid((const bf16*)dy, (const bf16*)y, r, nullptr, (bf16*)dx, N, D, s)
                             : Stream<float>::norm_bwd_resid((const float*)dy, (const float*)y, r, nullptr, (float*)dx, N, D, s);
}

int32_t femto_embed_gather(int32_t dtype, void* out, const void* table, const int32_t* tokens0, int32_t N, int32_t D,
                           int32_t rows, void* stream) {
  FEMTO_TRY(require_device());
  if (!out || !table || !tokens0 || N <= 0 || D <= 0 || rows <= 0) return femto_fail(FEMTO_ERR_ARG, "bad argument");
  if (dtype != FEMTO_F32 && dtype != FEMTO_BF16) return femto_fail(FEMTO_ERR_ARG, "dtype must be FEMTO_F32 or FEMTO_BF16");
  cudaStream_t s = (cudaStream_t)stream;
  unsigned int* status = nullptr;
  FEMTO_TRY(standalone_status(&status));
  const int grid = cdiv(N, 8);
  if (dtype == FEMTO_BF16) {
    if (D % 8 == 0 && aligned16(out) && aligned16(table)) k_embed_gather<bf16, 8><<<grid, 256, 0, s>>>((const bf16*)table, tokens0, (bf16*)out, N, D, rows, status);
    else k_embed_gather<bf16, 1><<<grid, 256, 0, s>>>((const bf16*)table, tokens0, (bf16*)out, N, D, rows, status);
  } else {
    if (D % 4 == 0 && aligned16(out) && aligned16(table)) k_embed_gather<float, 4><<<grid, 256, 0, s>>>((const float*)table, tokens0, (float*)out, N, D, rows, status);
    else k_embed_gather<float, 1><<<grid, 256, 0, s>>>((const float*)table, tokens0, (float*)out, N, D, rows, status);
  }
  KERNEL_CHECK();
  return 0;
}

int32_t femto_muon_direction(int32_t dtype, float* X_out, const float* G, float* momentum, float* second_moment,
                             int32_t k, int32_t rows, int32_t cols, float mu, float beta2, float n_tokens,
                             const float* h_coeffs, int32_t steps, void* stream) {
  FEMTO_TRY(require_device());
  if (!X_out || !G || !momentum || !second_moment || !h_coeffs || k <= 0 || rows <= 0 || cols <= 0 || steps < 0 || steps > 5)
    return femto_fail(FEMTO_ERR_ARG, "bad argument");
  if (!(n_tokens > 0.f)) return femto_fail(FEMTO_ERR_ARG, "n_tokens must be positive");
  if (dtype != FEMTO_F32 && dtype != FEMTO_BF16) return femto_fail(FEMTO_ERR_ARG, "dtype must be FEMTO_F32 or FEMTO_BF16");
  cudaStream_t s = (cudaStream_t)stream;
  unsigned int* status = nullptr;
  FEMTO_TRY(standalone_status(&status));
  int rc = muon_direction_standalone(dtype, X_out, G, momentum, second_moment, k, rows, cols, mu, beta2, n_tokens, h_coeffs,
                                     steps, status, s);
  return standalone_finish(rc, status, s);
}

int32_t femto_status_word(femto_handle* h, int32_t* out) {
  if (!out) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  unsigned int v = 0;
  if (!h) {
    // the stand-alone kernel-level entry points of the current device (synchronises the device)
    int dev = -1;
    CUDA_TRY(cudaGetDevice(&dev));
    CUDA_TRY(cudaDeviceSynchronize());
    if (dev >= 0 && dev < 64 && g_sa_status[dev]) {
      CUDA_TRY(cudaMemcpy(&v, g_sa_status[dev], sizeof(v), cudaMemcpyDeviceToHost));
      if (v) CUDA_TRY(cudaMemset(g_sa_status[dev], 0, sizeof(v)));   // read and clear
    }
    *out = (int32_t)(v | static_entry_status_word());
    return 0;
  }
  CUDA_TRY(cudaMemcpy(&v, h->status, sizeof(v), cudaMemcpyDeviceToHost));
  *out = (int32_t)v;
  return 0;
}

int32_t femto_sync(femto_handle* h, void* stream) {
  (void)h;
  CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
  return 0;
}

int64_t femto_launch_count(femto_handle* h) {
  (void)h;
  return g_femto_launches;
}

}  // extern "C"
