// Layout (src/parameters.jl:197-337), workspace arena and the forward / reverse schedule of the
// GPT step (src/gpt.jl:129-199; reverse rules ext/FemtoChatEnzymeExt.jl:69-204).
#include "model.cuh"

#include <math.h>
#include <stdarg.h>
#include <string.h>

#include <algorithm>

#include "streaming.cuh"

thread_local char g_femto_err[512] = {0};
long long g_femto_launches = 0;

int femto_fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_femto_err, sizeof(g_femto_err), fmt, ap);
  va_end(ap);
  return code;
}

// ---- layout -------------------------------------------------------------------------------------
static int check_cfg(const femto_config* c) {
  if (!c) return femto_fail(FEMTO_ERR_ARG, "config is NULL");
  if (c->n_embed <= 0 || c->n_head <= 0 || c->n_kv_head <= 0 || c->n_layer <= 0 || c->vocab_size <= 0 ||
      c->sequence_len <= 0 || c->max_document_tokens <= 0)
    return femto_fail(FEMTO_ERR_ARG, "config fields must be positive");
  if (c->n_embed % c->n_head != 0) return femto_fail(FEMTO_ERR_SHAPE, "n_embed %% n_head != 0");
  if (c->n_kv_head > c->n_head || c->n_head % c->n_kv_head != 0)
    return femto_fail(FEMTO_ERR_SHAPE, "n_head must be a multiple of n_kv_head");
  if ((c->n_embed / c->n_head) % 2 != 0) return femto_fail(FEMTO_ERR_SHAPE, "head_dim must be even (RoPE)");
  size_t pl = strnlen(c->window_pattern, sizeof(c->window_pattern));
  if (pl == 0 || pl >= sizeof(c->window_pattern)) return femto_fail(FEMTO_ERR_ARG, "window_pattern empty or unterminated");
  for (size_t i = 0; i < pl; i++)
    if (c->window_pattern[i] != 'S' && c->window_pattern[i] != 'L')
      return femto_fail(FEMTO_ERR_ARG, "window_pattern may hold only 'S' and 'L'");
  if (c->compute_dtype != FEMTO_F32 && c->compute_dtype != FEMTO_BF16)
    return femto_fail(FEMTO_ERR_ARG, "compute_dtype must be FEMTO_F32 or FEMTO_BF16");
  if (c->index_base != 0 && c->index_base != 1) return femto_fail(FEMTO_ERR_ARG, "index_base must be 0 or 1");
  return 0;
}

static bool has_ve(int layer1, int n_layer) { return (layer1 - 1) % 2 == (n_layer - 1) % 2; }

int layout_windows(const femto_config* c, std::vector<int>& left, std::vector<int>& ve) {
  FEMTO_TRY(check_cfg(c));
  const int L = c->sequence_len;
  int S = c->short_window > 0 ? std::min(L, c->short_window) : std::min(L, ((L + 511) / 512) * 128);
  const int pl = (int)strlen(c->window_pattern);
  left.assign(c->n_layer, L);
  ve.assign(c->n_layer, 0);
  for (int i = 0; i < c->n_layer; i++) {
    left[i] = c->window_pattern[i % pl] == 'S' ? S : L;
    ve[i] = has_ve(i + 1, c->n_layer) ? 1 : 0;
  }
  left[c->n_layer - 1] = L;
  return 0;
}

int layout_describe(const femto_config* c, std::vector<femto_tensor_desc>& out, long long* nparams, int* Vp_out) {
  FEMTO_TRY(check_cfg(c));
  const int pad = c->pad_vocab_size_to > 0 ? c->pad_vocab_size_to : 64;
  const long long d = c->n_embed, hd = d / c->n_head, kv = (long long)c->n_kv_head * hd;
  const long long Vp = ((c->vocab_size + pad - 1) / pad) * (long long)pad;
  long long pos = 0;
  out.clear();
  auto take = [&](int kind, int layer, long long rows, long long cols) {
    femto_tensor_desc t;
    t.kind = kind; t.layer = layer; t.offset = pos; t.rows = rows; t.cols = cols;
    pos += rows * cols;
    out.push_back(t);
  };
  take(0, -1, d, Vp);
  for (int i = 0; i < c->n_layer; i++) {
    const bool ve = has_ve(i + 1, c->n_layer);
    take(1, i, d, d);
    take(2, i, kv, d);
    take(3, i, kv, d);
    take(4, i, d, d);
    if (ve) take(5, i, c->n_kv_head, 12);
    take(6, i, 4 * d, d);
    take(7, i, d, 4 * d);
    if (ve) take(8, i, kv, Vp);
    take(9, i, 1, 1);
    take(10, i, 1, 1);
  }
  take(11, -1, Vp, d);
  take(12, -1, 1, 24);
  take(13, -1, 1, 1);
  take(14, -1, 1, 1);
  if (nparams) *nparams = pos;
  if (Vp_out) *Vp_out = (int)Vp;
  return 0;
}

int model_fill(femto_handle* h, const femto_config* cfg) {
  FEMTO_TRY(check_cfg(cfg));
  h->cfg = *cfg;
  if (h->cfg.pad_vocab_size_to <= 0) h->cfg.pad_vocab_size_to = 64;
  if (cfg->max_batch <= 0) return femto_fail(FEMTO_ERR_ARG, "max_batch must be positive");
  h->d = cfg->n_embed; h->H = cfg->n_head; h->Hkv = cfg->n_kv_head; h->hd = h->d / h->H;
  h->kv = h->Hkv * h->hd; h->dq = h->d + 2 * h->kv; h->V = cfg->vocab_size; h->L = cfg->n_layer;
  h->T = cfg->sequence_len; h->maxB = cfg->max_batch; h->maxN = h->maxB * h->T;
  h->bf = cfg->compute_dtype == FEMTO_BF16;
  h->eps = h->bf ? 0.0078125f : 1.1920929e-7f;  // eps(eltype(x)), src/gpt.jl:16
  if (h->d < 24) return femto_fail(FEMTO_ERR_SHAPE, "n_embed must be >= 24 (smear gate reads 24 channels)");
  std::vector<femto_tensor_desc> td;
  FEMTO_TRY(layout_describe(&h->cfg, td, &h->nparams, &h->Vp));
  std::vector<int> left, ve;
  FEMTO_TRY(layout_windows(&h->cfg, left, ve));
  h->lp.assign(h->L, LayerP());
  for (auto& l : h->lp) { l.ve_gate = -1; l.ve_table = -1; }
  for (const auto& t : td) {
    if (t.layer >= 0) {
      LayerP& l = h->lp[t.layer];
      switch (t.kind) {
        case 1: l.wq = t.offset; break;
        case 2: l.wk = t.offset; break;
        case 3: l.wv = t.offset; break;
        case 4: l.wo = t.offset; break;
        case 5: l.ve_gate = t.offset; break;
        case 6: l.fc = t.offset; break;
        case 7: l.proj = t.offset; break;
        case 8: l.ve_table = t.offset; break;
        case 9: l.lam_b = t.offset; break;
        case 10: l.lam_x0 = t.offset; break;
      }
    } else {
      switch (t.kind) {
        case 0: h->off_wte = t.offset; break;
        case 11: h->off_lm = t.offset; break;
        case 12: h->off_smear = t.offset; break;
        case 13: h->off_lam_s = t.offset; break;
        case 14: h->off_lam_y = t.offset; break;
      }
    }
  }
  for (int i = 0; i < h->L; i++) { h->lp[i].ve = ve[i] != 0; h->lp[i].window = left[i]; }
  h->backout = h->L / 2;  // 1-based n_layer/2+1 (src/gpt.jl:145)
  h->xchunk = std::min(h->maxN, 16384);
  return 0;
}

// ---- arena --------------------------------------------------------------------------------------
namespace {
struct Bump {
  char* base = nullptr;
  size_t off = 0;
  template <typename P> void take(P*& p, size_t bytes) {
    off = (off + 255) & ~(size_t)255;
    p = base ? reinterpret_cast<P*>(base + off) : nullptr;
    off += bytes;
  }
};

void carve(femto_handle* h, Bump& b) {
  const size_t es = h->bf ? 2 : 4;
  const size_t N = h->maxN, d = h->d, dq = h->dq, kv = h->kv, Vp = h->Vp;
  const size_t half = h->hd / 2;
  b.take(h->sin_t, sizeof(float) * h->cfg.max_document_tokens * half);
  b.take(h->cos_t, sizeof(float) * h->cfg.max_document_tokens * half);
  b.take(h->status, 256);
  // The compute-type copies of every weight lie in ONE contiguous range [weights_begin, weights_end): the
  // data-parallel update exchanges them with a single collective.
  h->lb.resize(h->L);
  b.take(h->sh_wte, es * Vp * d);
  h->weights_begin = reinterpret_cast<char*>(h->sh_wte);
  b.take(h->sh_lm, es * Vp * d);
  for (int i = 0; i < h->L; i++) {
    LayerBuf& l = h->lb[i];
    b.take(l.sh_wqkv, es * d * dq); b.take(l.sh_wo, es * d * d); b.take(l.sh_fc, es * d * 4 * d);
    b.take(l.sh_proj, es * 4 * d * d);
    if (h->lp[i].ve) b.take(l.sh_ve, es * Vp * kv); else l.sh_ve = nullptr;
  }
  { char* end = nullptr; b.take(end, 0); h->weights_end = end; }
  b.take(h->tok0, 4 * N); b.take(h->tgt0, 4 * N); b.take(h->pos, 4 * N); b.take(h->doc_start, 4 * N);
  b.take(h->raw_tok, 4 * N); b.take(h->raw_tgt, 4 * N); b.take(h->raw_pos, 4 * N);
  b.take(h->xe, es * N * d); b.take(h->x0, es * N * d); b.take(h->xm, es * N * d); b.take(h->xnf, es * N * d);
  b.take(h->sg, 4 * N); b.take(h->rf, 4 * N);
  for (int i = 0; i < h->L; i++) {
    LayerBuf& l = h->lb[i];
    b.take(l.xout, es * N * d); b.take(l.xn1, es * N * d); b.take(l.qkv, es * N * dq); b.take(l.att, es * N * d);
    b.take(l.xn2, es * N * d); b.take(l.a, es * N * 4 * d);
    b.take(l.r1, 4 * N); b.take(l.r2, 4 * N); b.take(l.rqk, 4 * N * (h->H + h->Hkv)); b.take(l.sv, 4 * N * h->Hkv);
    b.take(l.lse, 4 * N * h->H);
  }
  b.take(h->dx, es * N * d); b.take(h->dxn, es * N * d); b.take(h->dqkv, es * N * dq); b.take(h->datt, es * N * d);
  b.take(h->du, es * N * 4 * d); b.take(h->dx0, es * N * d); b.take(h->dxf, es * N * d); b.take(h->dve, es * N * kv);
  b.take(h->dx_b, es * N * d); b.take(h->dx_c, es * N * d); b.take(h->du_b, es * N * 4 * d); b.take(h->dqkv_b, es * N * dq);
  b.take(h->dpre, 4 * N * h->Hkv); b.take(h->dpre_s, 4 * N);
  b.take(h->partial, 4 * (size_t)std::max<size_t>(1024 * 32, (N / 256 + 1) * 12 * h->Hkv));
  const size_t xc = h->xchunk;
  if (!h->bf || 4 * xc * Vp <= ((size_t)512 << 20)) b.take(h->logits_f32, 4 * xc * Vp); else h->logits_f32 = nullptr;
  b.take(h->xstats, sizeof(float2) * xc * (2 * ((h->V + 255) / 256) + 2));
  b.take(h->tz, 4 * N); b.take(h->lse_rows, 4 * N); b.take(h->loss_rows, 4 * N); b.take(h->inv_nvalid, 256);
  b.take(h->dlogit, es * xc * Vp);
  b.take(h->dlogit_b, es * xc * Vp);
  b.take(h->loss_dev, 256); b.take(h->nvalid_dev, 256);
  h->gemm_ws_bytes = (size_t)160 << 20;
  b.take(h->gemm_ws, h->gemm_ws_bytes);
  b.take(h->gemm_ws2, h->gemm_ws_bytes);
  h->attn_ws_bytes = std::max(sizeof(float) * N * h->H * 2, attention_bwd_tc_ws_bytes(h->maxB, h->T, h->H, h->hd));
  b.take(h->attn_ws, h->attn_ws_bytes);
}

__global__ void k_rope_tables(float* sin_t, float* cos_t, int n, int half, int hd) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * half) return;
  int t = i / half, c = i % half;
  // inv_freq = 1 / base^(2c/hd), fp32 as in src/parameters.jl:424-425
  float inv = 1.f / powf(100000.f, (float)(2 * c) / (float)hd);
  float f = inv * (float)t;
  sin_t[i] = sinf(f);
  cos_t[i] = cosf(f);
}
}  // namespace

int model_alloc(femto_handle* h) {
  {
    // FEMTO_XENT_CHUNK in the environment overrides the lm_head tail's chunk of 16 384 tokens (256..32768; lets a
    // small test shape run the chunk loop with a ragged last chunk).  Measured: a chunk of 18 944 tokens, which makes
    // the dX product of a chunk a whole number of GEMM waves on 148 SMs, is no faster than 16 384.
    const char* env = getenv("FEMTO_XENT_CHUNK");
    if (env && atoi(env) >= 256 && atoi(env) <= 32768) h->xchunk = std::min(h->maxN, atoi(env) / 256 * 256);
  }
  Bump dry;
  carve(h, dry);
  h->arena_bytes = dry.off + 256;
  cudaError_t e = cudaMalloc(&h->arena, h->arena_bytes);
  if (e != cudaSuccess)
    return femto_fail(FEMTO_ERR_NOMEM, "cudaMalloc of %.2f GiB workspace failed: %s", h->arena_bytes / 1073741824.0,
                      cudaGetErrorString(e));
  Bump real;
  real.base = h->arena;
  carve(h, real);
  CUDA_TRY(cudaMemset(h->status, 0, 256));
  const int half = h->hd / 2, n = h->cfg.max_document_tokens;
  k_rope_tables<<<cdiv((long long)n * half, 256), 256>>>(h->sin_t, h->cos_t, n, half, h->hd);
  KERNEL_CHECK();
  int maxcols = std::max(h->d, h->kv);
  FEMTO_TRY(scatter_plan_create(&h->plan, h->maxN, maxcols));
  // FEMTO_SIDE_STREAM=0 in the environment keeps every launch on the caller's stream (measurement aid)
  const char* env = getenv("FEMTO_SIDE_STREAM");
  if (!(env && env[0] == '0')) {
    int least = 0, greatest = 0;
    CUDA_TRY(cudaDeviceGetStreamPriorityRange(&least, &greatest));
    CUDA_TRY(cudaStreamCreateWithPriority(&h->hi, cudaStreamNonBlocking, greatest));
    CUDA_TRY(cudaStreamCreateWithPriority(&h->lo, cudaStreamNonBlocking, least));
    for (auto& e : h->ev_fork) CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    for (auto& e : h->ev_side) CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  }
  CUDA_TRY(cudaDeviceSynchronize());
  return 0;
}

void model_free(femto_handle* h) {
  if (h->hi) { cudaStreamSynchronize(h->hi); cudaStreamDestroy(h->hi); h->hi = nullptr; }
  if (h->lo) { cudaStreamSynchronize(h->lo); cudaStreamDestroy(h->lo); h->lo = nullptr; }
  for (auto& e : h->ev_fork) if (e) { cudaEventDestroy(e); e = nullptr; }
  for (auto& e : h->ev_side) if (e) { cudaEventDestroy(e); e = nullptr; }
  if (h->plan) scatter_plan_destroy(h->plan);
  h->plan = nullptr;
  if (h->arena) cudaFree(h->arena);
  h->arena = nullptr;
}

template <typename T> static int refresh_t(femto_handle* h, const float* theta, cudaStream_t s) {
  const long long d = h->d, Vp = h->Vp, kv = h->kv;
  FEMTO_TRY(Stream<T>::cast_from_f32(theta + h->off_wte, (T*)h->sh_wte, Vp * d, s));
  FEMTO_TRY(Stream<T>::cast_from_f32(theta + h->off_lm, (T*)h->sh_lm, Vp * d, s));
  for (int i = 0; i < h->L; i++) {
    const LayerP& p = h->lp[i];
    LayerBuf& l = h->lb[i];
    FEMTO_TRY(Stream<T>::pack_qkv(theta + p.wq, theta + p.wk, theta + p.wv, (T*)l.sh_wqkv, h->d, h->kv, s));
    FEMTO_TRY(Stream<T>::cast_from_f32(theta + p.wo, (T*)l.sh_wo, d * d, s));
    FEMTO_TRY(Stream<T>::cast_from_f32(theta + p.fc, (T*)l.sh_fc, 4 * d * d, s));
    FEMTO_TRY(Stream<T>::cast_from_f32(theta + p.proj, (T*)l.sh_proj, 4 * d * d, s));
    if (p.ve) FEMTO_TRY(Stream<T>::cast_from_f32(theta + p.ve_table, (T*)l.sh_ve, Vp * kv, s));
  }
  h->weights_valid = true;
  return 0;
}

int model_refresh(femto_handle* h, const float* theta, cudaStream_t s) {
  return h->bf ? refresh_t<bf16>(h, theta, s) : refresh_t<float>(h, theta, s);
}

// ---- forward / reverse schedule --------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(1024) k_inv_nvalid(const int* tgt0, int n, float* out) {
  __shared__ int red[32];
  int c = 0;
  for (int i = threadIdx.x; i < n; i += 1024) c += tgt0[i] >= 0 ? 1 : 0;
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int i = 0; i < 32; i++) t += red[i];
    out[0] = 1.f / (float)t;
  }
}
}  // namespace

template <typename T>
static int step_t(femto_handle* h, const float* theta, float* delta, const int* tokens, const int* targets,
                  const int* positions, int B, int reduction, bool backward, bool accumulate, float* loss_out,
                  int* nvalid_out, cudaStream_t s, cudaStream_t side, float* logits_out, float* token_losses_out,
                  const StepExtra* ex) {
  typedef Stream<T> S;
  const int Tl = (ex && ex->T > 0) ? ex->T : h->T;
  const int N = B * Tl, d = h->d, dq = h->dq, kv = h->kv, H = h->H, Hkv = h->Hkv, hd = h->hd, Vp = h->Vp, V = h->V;
  const int L = h->L;
  const float eps = h->eps;
  const bool mean = reduction == FEMTO_REDUCTION_MEAN;
  // with a side stream the GEMMs give up one ring stage (32 KB), so that streaming kernels of the other stream fit beside them
  auto GA = [&]() { GemmArgs g; g.ws = h->gemm_ws; g.ws_bytes = h->gemm_ws_bytes; g.status = h->status; g.ring = (backward && side) ? 5 : 0; return g; };
  // Y[N][out] = X[N][in] * W[in][out]
  auto lin_fwd = [&](const void* X, int in, const void* W, int out, void* Y, int ldy, int epi, const void* aux) {
    GemmArgs g = GA();
    g.A = X; g.lda = in; g.a_kmajor = true; g.B = W; g.ldb = out; g.b_kmajor = false;
    g.C = Y; g.ldc = ldy; g.M = N; g.N = out; g.K = in; g.epi = epi; g.aux = aux; g.ldaux = ldy;
    return gemm<T>(g, s);
  };
  // dX[N][in] = dY[N][out] * W[in][out]^T
  auto lin_dx = [&](const void* dY, int ldy, int out, const void* W, int in, void* dX, int epi, const void* aux) {
    GemmArgs g = GA();
    g.A = dY; g.lda = ldy; g.a_kmajor = true; g.B = W; g.ldb = out; g.b_kmajor = true;
    g.C = dX; g.ldc = in; g.M = N; g.N = in; g.K = out; g.epi = epi; g.aux = aux; g.ldaux = in;
    return gemm<T>(g, s);
  };
  // The weight-gradient GEMMs, the zero fill of delta: on the side stream when the handle has one (`s` is then the
  // handle's chain stream).  fork(): the side stream waits for everything queued on the chain so far.
  // side_read(slot): the side stream's last launch read gradient buffer `slot`; chain_write(slot): the chain is
  // about to overwrite that buffer and waits for that reader.
  cudaStream_t s2 = (backward && side) ? side : s;
  const bool two = s2 != s;
  enum { SL_DX = 0, SL_DU = 3, SL_DQKV = 5, SL_FILL = 7, SL_DVE = 10 };   // 8, 9: the lm_head tail's two d-logit buffers
  auto fork = [&]() -> int {
    if (!two) return 0;
    cudaEvent_t e = h->ev_fork[h->ev_next++ % femto_handle::N_FORK];
    CUDA_TRY(cudaEventRecord(e, s));
    CUDA_TRY(cudaStreamWaitEvent(s2, e, 0));
    return 0;
  };
  auto side_read = [&](int slot) -> int {
    if (!two) return 0;
    CUDA_TRY(cudaEventRecord(h->ev_side[slot], s2));
    h->side_armed[slot] = true;
    return 0;
  };
  auto chain_write = [&](int slot) -> int {
    if (!two || !h->side_armed[slot]) return 0;
    CUDA_TRY(cudaStreamWaitEvent(s, h->ev_side[slot], 0));
    h->side_armed[slot] = false;
    return 0;
  };
  auto join = [&]() -> int {   // the chain waits for everything queued on the side stream
    if (!two) return 0;
    cudaEvent_t e = h->ev_fork[h->ev_next++ % femto_handle::N_FORK];
    CUDA_TRY(cudaEventRecord(e, s2));
    CUDA_TRY(cudaStreamWaitEvent(s, e, 0));
    for (bool& a : h->side_armed) a = false;
    return 0;
  };
  // dW[in][out] += X[N][in]^T * dY[N][out]
  auto lin_dw = [&](const void* X, int in, const void* dY, int ldy, int out, float* dW) {
    GemmArgs g = GA();
    if (two) g.ws = h->gemm_ws2;
    g.A = X; g.lda = in; g.a_kmajor = false; g.B = dY; g.ldb = ldy; g.b_kmajor = false;
    g.C = dW; g.ldc = out; g.M = in; g.N = out; g.K = N; g.epi = EPI_F32; g.beta = accumulate ? 1.f : 0.f;
    return gemm<T>(g, s2);
  };

  FEMTO_TRY(S::prep_tokens(tokens, targets, positions, B, Tl, h->cfg.index_base, V, h->cfg.max_document_tokens,
                           h->tok0, h->tgt0, h->pos, h->doc_start, h->status, s));
  // A step that does not accumulate overwrites the matrices' ranges of delta (their products run with beta = 0) and
  // zero-fills only what is summed into: the embedding tables (row scatter), the gates and the scalars.  Off the
  // chain: nothing reads or writes delta before the lm_head tail.
  const bool lm_overwrite = V == Vp;   // padding columns of lm_head are written by nobody: keep the fill for them
  if (backward && !accumulate) {
    FEMTO_TRY(fork());
    auto zero = [&](long long off, long long n) { return n > 0 ? fill_zero(delta + off, sizeof(float) * (size_t)n, s2) : 0; };
    FEMTO_TRY(zero(h->off_wte, (long long)Vp * d));
    for (int i = 0; i < L; i++) {
      const LayerP& p = h->lp[i];
      if (p.ve) FEMTO_TRY(zero(p.ve_gate, 12ll * Hkv));
      const long long from = p.ve ? p.ve_table : p.lam_b;
      FEMTO_TRY(zero(from, p.lam_x0 + 1 - from));
    }
    if (!lm_overwrite) FEMTO_TRY(zero(h->off_lm, (long long)Vp * d));
    FEMTO_TRY(zero(h->off_smear, h->nparams - h->off_smear));
    FEMTO_TRY(side_read(SL_FILL));
  }
  const int* docs = h->cfg.doc_mask ? h->doc_start : nullptr;

  // ---- forward (src/gpt.jl:129-170) ----
  FEMTO_TRY(S::embed_norm((const T*)h->sh_wte, h->tok0, (T*)h->xe, N, d, eps, s));
  FEMTO_TRY(S::smear((const T*)h->xe, theta + h->off_smear, theta + h->off_lam_s, N, Tl, d, h->sg, (T*)h->x0, s));
  for (int i = 0; i < L; i++) {
    const LayerP& p = h->lp[i];
    LayerBuf& l = h->lb[i];
    const T* xin = i == 0 ? (const T*)h->x0 : (const T*)h->lb[i - 1].xout;
    FEMTO_TRY(S::mix_norm(xin, (const T*)h->x0, theta + p.lam_b, theta + p.lam_x0, (T*)h->xm, (T*)l.xn1, l.r1, N, d, eps, s));
    FEMTO_TRY(lin_fwd(l.xn1, d, l.sh_wqkv, dq, l.qkv, dq, EPI_STORE, nullptr));
    FEMTO_TRY(S::qkv_post((T*)l.qkv, dq, (const T*)l.xn1, d, p.ve ? theta + p.ve_gate : nullptr,
                          p.ve ? (const T*)l.sh_ve : nullptr, h->tok0, h->pos, h->sin_t, h->cos_t, N, H, Hkv, hd, eps,
                          l.rqk, l.sv, s));
    AttnArgs a;
    a.Q = l.qkv; a.K = (const T*)l.qkv + d; a.V = (const T*)l.qkv + d + kv; a.q_stride = dq; a.kv_stride = dq;
    a.O = l.att; a.o_stride = d; a.lse = l.lse; a.B = B; a.T = Tl; a.H = H; a.Hkv = Hkv; a.hd = hd;
    a.window_left = p.window; a.doc_start = docs; a.ws = h->attn_ws; a.ws_bytes = h->attn_ws_bytes; a.status = h->status;
    FEMTO_TRY(attention_fwd<T>(a, s));
    FEMTO_TRY(lin_fwd(l.att, d, l.sh_wo, d, h->xm, d, EPI_RESID, h->xm));
    FEMTO_TRY(S::norm((const T*)h->xm, (T*)l.xn2, l.r2, N, d, eps, s));
    FEMTO_TRY(lin_fwd(l.xn2, d, l.sh_fc, 4 * d, l.a, 4 * d, EPI_RELU2, nullptr));
    {
      GemmArgs g = GA();
      g.A = l.a; g.lda = 4 * d; g.B = l.sh_proj; g.ldb = d; g.b_kmajor = false; g.C = l.xout; g.ldc = d;
      g.M = N; g.N = d; g.K = 4 * d; g.epi = EPI_RESID; g.aux = h->xm; g.ldaux = d;
      FEMTO_TRY(gemm<T>(g, s));
    }
  }
  const T* xlast = (const T*)h->lb[L - 1].xout;
  const T* xb = (const T*)h->lb[h->backout].xout;
  FEMTO_TRY(S::backout_norm(xlast, xb, theta + h->off_lam_y, nullptr, (T*)h->xnf, h->rf, N, d, eps, s));

  // ---- a prompt: its keys / values go to the cache, and only the last position of each column needs logits ----
  if (ex && ex->cache) {
    FEMTO_TRY(kv_cache_store_prompt<T>(ex->cache, B, Tl, s));
    return kv_cache_last_logits<T>(ex->cache, (const T*)h->xnf, B, Tl, ex->last_logits, s);
  }

  // ---- the model call without targets returns the soft-capped logits of the first V rows (src/gpt.jl:165-170) ----
  if (logits_out) {
    GemmArgs g = GA();
    g.A = h->xnf; g.lda = d; g.a_kmajor = true; g.B = h->sh_lm; g.ldb = Vp; g.b_kmajor = false;
    g.C = logits_out; g.ldc = V; g.M = N; g.N = V; g.K = d; g.epi = EPI_F32; g.beta = 0.f;
    FEMTO_TRY(gemm<T>(g, s));
    return softcap_inplace(logits_out, (long long)N * V, s);
  }

  // ---- lm_head tail (src/gpt.jl:165-194), token chunks; reverse fused in (src/kernels.jl:16-28) ----
  if (mean) {
    k_inv_nvalid<<<1, 1024, 0, s>>>(h->tgt0, N, h->inv_nvalid);
    KERNEL_CHECK();
  }
  T* dxnf = (T*)h->dxn;
  {
    XentArgs x;
    x.x = h->xnf; x.W = h->sh_lm; x.ldw = Vp; x.targets0 = h->tgt0; x.N = N; x.D = d; x.V = V;
    x.scale_dev = mean ? h->inv_nvalid : nullptr; x.backward = backward; x.dx = dxnf;
    x.dw = backward ? delta + h->off_lm : nullptr; x.chunk = h->xchunk; x.logits_f32 = h->logits_f32;
    x.dw_overwrite = backward && !accumulate && lm_overwrite;
    x.stats = h->xstats; x.tz = h->tz; x.lse_rows = h->lse_rows; x.loss_rows = h->loss_rows; x.dlogit = h->dlogit;
    x.ws = h->gemm_ws; x.ws_bytes = h->gemm_ws_bytes; x.status = h->status;
    if (two) {
      x.side = s2; x.ws2 = h->gemm_ws2; x.dlogit2 = h->dlogit_b;
      x.ev_read[0] = h->ev_side[8]; x.ev_read[1] = h->ev_side[9];
      x.ev_fork[0] = h->ev_fork[h->ev_next++ % femto_handle::N_FORK];
      x.ev_fork[1] = h->ev_fork[h->ev_next++ % femto_handle::N_FORK];
    }
    FEMTO_TRY(xent_tail<T>(x, s));
  }
  if (token_losses_out)   // reduction=:none (src/gpt.jl:191-193): one loss per token slot, 0 where the target is ignored
    CUDA_TRY(cudaMemcpyAsync(token_losses_out, h->loss_rows, sizeof(float) * (size_t)N, cudaMemcpyDeviceToDevice, s));
  if (loss_out) FEMTO_TRY(sum_rows_to_scalar(h->loss_rows, N, loss_out, h->tgt0, nvalid_out, mean ? 1.f : 0.f, s));
  if (!backward) return 0;

  // ---- reverse ----
  // With overlap_sync each finished range of delta (lm_head, then one transformer block at a time,
  // then the embeddings) is summed over ranks on the communication stream while the rest of the
  // reverse pass runs.
  const bool ov = h->overlap_sync && h->dp != nullptr;
  h->delta_synced = false;
  FEMTO_TRY(chain_write(SL_FILL));   // the chain's first write into delta follows the zero fill
  if (ov) {
    FEMTO_TRY(join());
    FEMTO_TRY(dp_bucket_allreduce(h->dp, delta + h->off_lm, (long long)Vp * d, s));
  }
  int nb = 0;
  FEMTO_TRY(scatter_plan_build(h->plan, h->tok0, N, Vp, s));
  FEMTO_TRY(S::head_bwd(dxnf, (const T*)h->xnf, h->rf, xb, (T*)h->dxf, N, d, h->partial, &nb, s));
  FEMTO_TRY(reduce_partials(h->partial, nb, 1, delta + h->off_lam_y, nullptr, 1.f, true, s));
  // The gradient of the residual stream rotates through three buffers, d(MLP pre-activation) and d(QKV) through
  // two each: a weight-gradient GEMM on the side stream may still be reading one while the chain writes the next.
  // The last block reads its incoming gradient straight from dxf (nothing writes dxf again in this step).
  T* dxr[3] = {(T*)h->dx, (T*)h->dx_b, (T*)h->dx_c};
  T* dur[2] = {(T*)h->du, (T*)h->du_b};
  T* dqr[2] = {(T*)h->dqkv, (T*)h->dqkv_b};
  T* dx = (T*)h->dxf;
  int cs = -1, nf = 0;   // hazard slot of dx (-1: dxf, no slot) and the next free buffer of the rotation
  T* dxn = (T*)h->dxn;
  for (int i = L - 1; i >= 0; i--) {
    const LayerP& p = h->lp[i];
    LayerBuf& l = h->lb[i];
    const T* xin = i == 0 ? (const T*)h->x0 : (const T*)h->lb[i - 1].xout;
    const int c1 = nf, c2 = (nf + 1) % 3, par = i & 1;
    T *dx1 = dxr[c1], *dx2 = dxr[c2], *du = dur[par], *dqkv = dqr[par];
    if (i == h->backout) {
      if (cs < 0) {   // a model so shallow that the backout block is the last one: work on a copy, dxf is the operand
        CUDA_TRY(cudaMemcpyAsync(dxr[2], h->dxf, sizeof(T) * (size_t)N * d, cudaMemcpyDeviceToDevice, s));
        dx = dxr[2]; cs = 2;
      }
      FEMTO_TRY(S::axpy(dx, (const T*)h->dxf, theta + h->off_lam_y, -1.f, (long long)N * d, s));
    }
    // MLP (ext/FemtoChatEnzymeExt.jl:121-134)
    FEMTO_TRY(fork());
    FEMTO_TRY(lin_dw(l.a, 4 * d, dx, d, d, delta + p.proj));
    if (cs >= 0) FEMTO_TRY(side_read(SL_DX + cs));
    FEMTO_TRY(chain_write(SL_DU + par));
    FEMTO_TRY(lin_dx(dx, d, d, l.sh_proj, 4 * d, du, EPI_DRELU2, l.a));
    FEMTO_TRY(fork());
    FEMTO_TRY(lin_dw(l.xn2, d, du, 4 * d, 4 * d, delta + p.fc));
    FEMTO_TRY(side_read(SL_DU + par));
    FEMTO_TRY(lin_dx(du, 4 * d, 4 * d, l.sh_fc, d, dxn, EPI_STORE, nullptr));
    FEMTO_TRY(chain_write(SL_DX + c1));
    FEMTO_TRY(S::norm_bwd_resid(dxn, (const T*)l.xn2, l.r2, dx, dx1, N, d, s));
    // attention block
    FEMTO_TRY(fork());
    FEMTO_TRY(lin_dw(l.att, d, dx1, d, d, delta + p.wo));
    FEMTO_TRY(side_read(SL_DX + c1));
    FEMTO_TRY(lin_dx(dx1, d, d, l.sh_wo, d, h->datt, EPI_STORE, nullptr));
    FEMTO_TRY(chain_write(SL_DQKV + par));
    AttnArgs a;
    a.Q = l.qkv; a.K = (const T*)l.qkv + d; a.V = (const T*)l.qkv + d + kv; a.q_stride = dq; a.kv_stride = dq;
    a.O = l.att; a.o_stride = d; a.lse = l.lse; a.dO = h->datt; a.do_stride = d;
    a.dQ = dqkv; a.dK = dqkv + d; a.dV = dqkv + d + kv; a.dq_stride = dq; a.dkv_stride = dq;
    a.B = B; a.T = Tl; a.H = H; a.Hkv = Hkv; a.hd = hd; a.window_left = p.window; a.doc_start = docs;
    a.ws = h->attn_ws; a.ws_bytes = h->attn_ws_bytes; a.status = h->status;
    FEMTO_TRY(attention_bwd<T>(a, s));
    if (p.ve) FEMTO_TRY(chain_write(SL_DVE));   // the previous value-embedding scatter has read dve
    FEMTO_TRY(S::qkv_post_bwd(dqkv, (const T*)l.qkv, dq, p.ve ? (const T*)l.sh_ve : nullptr, h->tok0, h->pos,
                              h->sin_t, h->cos_t, N, H, Hkv, hd, l.rqk, l.sv, (T*)h->dve, h->dpre, s));
    FEMTO_TRY(fork());
    {
      GemmArgs g = GA();  // fused dW of Q, K, V: three destinations in delta
      if (two) g.ws = h->gemm_ws2;
      g.A = l.xn1; g.lda = d; g.a_kmajor = false; g.B = dqkv; g.ldb = dq; g.b_kmajor = false;
      g.M = d; g.N = dq; g.K = N; g.epi = EPI_F32; g.beta = accumulate ? 1.f : 0.f; g.nseg = 3;
      g.seg_col0[0] = 0; g.seg_ncol[0] = d; g.seg_ptr[0] = delta + p.wq; g.seg_ld[0] = d;
      g.seg_col0[1] = d; g.seg_ncol[1] = kv; g.seg_ptr[1] = delta + p.wk; g.seg_ld[1] = kv;
      g.seg_col0[2] = d + kv; g.seg_ncol[2] = kv; g.seg_ptr[2] = delta + p.wv; g.seg_ld[2] = kv;
      g.C = delta + p.wq; g.ldc = d;
      FEMTO_TRY(gemm<T>(g, s2));
    }
    FEMTO_TRY(side_read(SL_DQKV + par));
    FEMTO_TRY(lin_dx(dqkv, dq, dq, l.sh_wqkv, d, dxn, EPI_STORE, nullptr));
    if (p.ve) {
      FEMTO_TRY(S::ve_gate_bwd((const T*)l.xn1, d, h->dpre, theta + p.ve_gate, dxn, N, Hkv, h->partial, &nb, s));
      FEMTO_TRY(reduce_partials(h->partial, nb, 12 * Hkv, delta + p.ve_gate, nullptr, 1.f, true, s));
      // the row scatter into the value-embedding table's gradient: nothing on the chain waits for it
      FEMTO_TRY(fork());
      FEMTO_TRY(scatter_rows<T>(h->plan, delta + p.ve_table, (const T*)h->dve, kv, kv, s2));
      FEMTO_TRY(side_read(SL_DVE));
    }
    FEMTO_TRY(chain_write(SL_DX + c2));
    FEMTO_TRY(S::mix_bwd(dx1, dx2, dxn, (const T*)l.xn1, l.r1, xin, (const T*)h->x0, theta + p.lam_b, theta + p.lam_x0,
                         (T*)h->dx0, i == L - 1, N, d, h->partial, &nb, s));
    FEMTO_TRY(reduce_partials(h->partial, nb, 2, delta + p.lam_b, nullptr, 1.f, true, s));
    dx = dx2; cs = c2; nf = (c2 + 1) % 3;
    if (ov) {
      FEMTO_TRY(join());
      FEMTO_TRY(dp_bucket_allreduce(h->dp, delta + p.wq, p.lam_x0 + 1 - p.wq, s));   // the block's range is contiguous
    }
  }
  FEMTO_TRY(S::add((T*)h->dx0, dx, (long long)N * d, s));
  FEMTO_TRY(S::smear_gate_bwd((const T*)h->dx0, (const T*)h->xe, h->sg, theta + h->off_lam_s, N, Tl, d, h->dpre_s,
                              h->partial, &nb, s));
  FEMTO_TRY(reduce_partials(h->partial, nb, 25, delta + h->off_smear, nullptr, 1.f, true, s));
  FEMTO_TRY(S::embed_bwd((const T*)h->dx0, (const T*)h->sh_wte, h->tok0, (const T*)h->xe, h->sg, h->dpre_s,
                         theta + h->off_smear, theta + h->off_lam_s, N, Tl, d, eps, dxn, s));
  FEMTO_TRY(fork());
  FEMTO_TRY(scatter_rows<T>(h->plan, delta + h->off_wte, dxn, d, d, s2));
  FEMTO_TRY(join());
  if (ov) {
    FEMTO_TRY(dp_bucket_allreduce(h->dp, delta + h->off_wte, (long long)Vp * d, s));
    FEMTO_TRY(dp_bucket_allreduce(h->dp, delta + h->off_smear, 26, s));   // smear gate (24), lam_s, lam_y
    h->delta_synced = true;
  }
  return 0;
}

int model_step(femto_handle* h, const float* theta, float* delta, const int* tokens, const int* targets,
               const int* positions, int B, int reduction, bool backward, bool accumulate, float* loss_out,
               int* nvalid_out, cudaStream_t s, float* logits_out, float* token_losses_out, const StepExtra* ex) {
  const bool prompt = ex && ex->cache && ex->last_logits;
  if (!h || !theta || !tokens || (!logits_out && !prompt && (!targets || (!loss_out && !token_losses_out))))
    return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  if (ex && ex->T > 0 && (long long)B * ex->T > h->maxN) return femto_fail(FEMTO_ERR_SHAPE, "B x T = %d x %d exceeds the workspace", B, ex->T);
  if (ex && ex->T > 0 && ex->T != h->T && backward) return femto_fail(FEMTO_ERR_UNSUPPORTED, "the reverse pass runs at sequence_len only");
  if (backward && !delta) return femto_fail(FEMTO_ERR_ARG, "delta is NULL");
  if (B <= 0 || B > h->maxB) return femto_fail(FEMTO_ERR_SHAPE, "B=%d outside 1..max_batch=%d", B, h->maxB);
  if (reduction != FEMTO_REDUCTION_SUM && reduction != FEMTO_REDUCTION_MEAN)
    return femto_fail(FEMTO_ERR_ARG, "reduction must be FEMTO_REDUCTION_SUM or FEMTO_REDUCTION_MEAN");
  if (!h->weights_valid) return femto_fail(FEMTO_ERR_STATE, "call femto_refresh_weights before the first step");
  if (!aligned16(theta) || (delta && !aligned16(delta))) return femto_fail(FEMTO_ERR_ALIGN, "Theta/delta must be 16-byte aligned");
  // A training step runs on the handle's own two streams, bracketed by the caller's stream on both sides; every
  // other call (loss only, logits, a prompt) is one dependency chain and stays on the caller's stream.
  const bool two = backward && h->hi && h->lo && !gemm_profiling();
  cudaStream_t chain = two ? h->hi : s;
  if (two) {
    cudaEvent_t e = h->ev_fork[h->ev_next++ % femto_handle::N_FORK];
    CUDA_TRY(cudaEventRecord(e, s));
    CUDA_TRY(cudaStreamWaitEvent(chain, e, 0));
  }
  const int r = h->bf ? step_t<bf16>(h, theta, delta, tokens, targets, positions, B, reduction, backward, accumulate,
                                     loss_out, nvalid_out, chain, two ? h->lo : nullptr, logits_out, token_losses_out, ex)
                      : step_t<float>(h, theta, delta, tokens, targets, positions, B, reduction, backward, accumulate,
                                      loss_out, nvalid_out, chain, two ? h->lo : nullptr, logits_out, token_losses_out, ex);
  if (two) {   // also after an error: whatever was queued is ordered before the caller's next work
    cudaEvent_t e = h->ev_fork[h->ev_next++ % femto_handle::N_FORK];
    cudaEventRecord(e, h->lo);
    cudaStreamWaitEvent(chain, e, 0);
    cudaEvent_t e2 = h->ev_fork[h->ev_next++ % femto_handle::N_FORK];
    cudaEventRecord(e2, chain);
    cudaStreamWaitEvent(s, e2, 0);
    for (bool& a : h->side_armed) a = false;
  }
  return r;
}
