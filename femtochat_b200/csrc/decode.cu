// Generation with a key/value cache.  The reference recomputes the whole context for every new token
// (src/generation.jl:26-56; "TODO" at src/gpt.jl:81): here the prompt is run once through the ordinary forward
// pass, which leaves the post-RoPE, post-QK-norm keys and the gated values of every block in a per-layer cache,
// and each further token runs a one-row-per-column forward (src/gpt.jl:129-170) whose attention reads that cache.
// The decode step is bound by HBM: every weight is read once per token, so the matrix products are a
// weight-streaming kernel (no tensor cores: M is the number of batch columns) and attention is a split-key kernel.
#include <algorithm>
#include <vector>

#include "model.cuh"
#include "streaming.cuh"

struct femto_kv_cache {
  femto_handle* h = nullptr;
  int maxB = 0, maxT = 0, B = 0, len = 0;     // len: tokens cached per column (all columns alike)
  char* mem = nullptr;
  std::vector<void*> K, V;                    // per block: [maxB][maxT][kv] of the compute type
  void* xe_prev = nullptr;                    // [maxB][d] normalised embedding of the last token (smear)
  void* xe_new = nullptr;                     // [maxB][d]
  int *tok0 = nullptr, *pos = nullptr, *doc_start = nullptr, *lastpos = nullptr;   // [maxB]
  float* part = nullptr;                      // split-key partials of the decode attention / split-K of the products
  size_t part_floats = 0;
};

namespace {

constexpr int MAX_SPLITS = 32;

// tok0 / pos / doc_start of the new token of every column.  positions == NULL continues each column's document:
// position = last position + 1 (the reference passes first_token-1 : length-1, src/generation.jl:47-48).
__global__ void k_decode_prep(const int* tokens, const int* positions, int B, int base, int vocab, int maxdoc, int len,
                              int* tok0, int* pos, int* doc_start, int* lastpos, unsigned int* status) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  int tk = tokens[b] - base;
  if (tk < 0 || tk >= vocab) { atomicOr(status, ST_BAD_TOKEN); tk = min(max(tk, 0), vocab - 1); }
  tok0[b] = tk;
  int p = positions ? positions[b] : lastpos[b] + 1;
  if (p < 0 || p >= maxdoc) { atomicOr(status, ST_BAD_TOKEN); p = min(max(p, 0), maxdoc - 1); }
  pos[b] = p;
  lastpos[b] = p;
  doc_start[b] = max(0, len - p);   // index (within the column) of the first token of this token's document
}

// x0 = xe + lam_s * sigmoid(w . xe[0:24]) * xe_prev (src/gpt.jl:118-122,139-140), same operation order as the
// full-sequence kernel; then xe becomes the new xe_prev.  One warp per column.
template <typename T>
__global__ void __launch_bounds__(256) k_smear_decode(const T* __restrict__ xe, T* __restrict__ xe_prev,
                                                      const float* __restrict__ w_s, const float* __restrict__ lam_s,
                                                      int B, int D, T* __restrict__ x0) {
  const int lane = threadIdx.x & 31;
  const int b = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (b >= B) return;
  const T* cur = xe + (long long)b * D;
  T* prev = xe_prev + (long long)b * D;
  float pre = lane < 24 ? to_f<T>(cur[lane]) * w_s[lane] : 0.f;
  pre = warp_sum(pre);
  const float gate = lam_s[0] * (1.f / (1.f + expf(-pre)));
  for (int c = lane; c < D; c += 32) {
    const float f = to_f<T>(cur[c]);
    x0[(long long)b * D + c] = from_f<T>(f + gate * to_f<T>(prev[c]));
    prev[c] = cur[c];
  }
}

// K / V of the new token (columns d.. and d+kv.. of its packed QKV row) go to row `t` of the block's cache.
template <typename T>
__global__ void k_kv_append(const T* __restrict__ qkv, long long ldq, int d, int kv, T* __restrict__ Kc, T* __restrict__ Vc,
                            int maxT, int t, int B) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)B * kv) return;
  const int b = (int)(i / kv), c = (int)(i % kv);
  const T* row = qkv + (long long)b * ldq;
  Kc[((long long)b * maxT + t) * kv + c] = row[d + c];
  Vc[((long long)b * maxT + t) * kv + c] = row[d + kv + c];
}
// The prompt's K / V rows [B][Tp] of one block into the cache.
template <typename T>
__global__ void k_kv_prefill(const T* __restrict__ qkv, long long ldq, int d, int kv, T* __restrict__ Kc, T* __restrict__ Vc,
                             int maxT, int Tp, int B) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)B * Tp * kv) return;
  const int c = (int)(i % kv);
  const long long bt = i / kv;
  const int b = (int)(bt / Tp), t = (int)(bt % Tp);
  const T* row = qkv + bt * ldq;
  Kc[((long long)b * maxT + t) * kv + c] = row[d + c];
  Vc[((long long)b * maxT + t) * kv + c] = row[d + kv + c];
}
template <typename T>
__global__ void k_take_last_rows(const T* __restrict__ x, int Tp, int D, int B, T* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)B * D) return;
  const int b = (int)(i / D), c = (int)(i % D);
  out[i] = x[((long long)b * Tp + Tp - 1) * D + c];
}
__global__ void k_take_last_pos(const int* pos, int Tp, int B, int* lastpos) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) lastpos[b] = pos[(long long)b * Tp + Tp - 1];
}

// ---- decode attention ------------------------------------------------------------------------------------------
// One query per (column, head) against the cached keys lo..tq of its kv head (tq = the new token's own row):
// softmax(q . k / sqrt(hd)) v in fp32 (src/kernels.jl:59-96 for a single query row).  grid (Hkv, B, splits): a
// block of four warps takes one contiguous range of keys; a warp takes every fourth key of it, each lane PER
// contiguous channels, and serves all G = H / Hkv query heads of the group from one load of the key and value rows.
// Partials (max, sum, unnormalised output) are combined over warps in shared memory and over splits by
// k_decode_attn_combine in split order, so the result does not depend on scheduling.
template <typename T, int PER, int GMAX>
__global__ void __launch_bounds__(128) k_decode_attn(const T* __restrict__ qkv, long long ldq, const T* __restrict__ Kc,
                                                     const T* __restrict__ Vc, int maxT, int kv, int tq, int window_left,
                                                     const int* __restrict__ doc_start, int H, int Hkv, int hd,
                                                     float* __restrict__ part, int splits) {
  const int kvh = blockIdx.x, b = blockIdx.y, sp = blockIdx.z;
  const int G = H / Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int lo = max(0, tq - window_left);
  if (doc_start) lo = max(lo, doc_start[b]);
  const int nkeys = tq - lo + 1;
  const int per_split = (nkeys + splits - 1) / splits;
  const int k_begin = lo + sp * per_split, k_end = min(tq + 1, k_begin + per_split);
  const float scale = rsqrtf((float)hd);
  float q[GMAX][PER], o[GMAX][PER], m[GMAX], l[GMAX];
  const bool lane_ok = lane * PER < hd;
#pragma unroll
  for (int g = 0; g < GMAX; g++) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < PER; e++) {
      o[g][e] = 0.f;
      q[g][e] = (g < G && lane_ok) ? to_f<T>(qkv[(long long)b * ldq + (long long)(kvh * G + g) * hd + lane * PER + e]) : 0.f;
    }
  }
  for (int k = k_begin + warp; k < k_end; k += 4) {
    const T* kr = Kc + ((long long)b * maxT + k) * kv + (long long)kvh * hd + lane * PER;
    const T* vr = Vc + ((long long)b * maxT + k) * kv + (long long)kvh * hd + lane * PER;
    float kf[PER], vf[PER];
#pragma unroll
    for (int e = 0; e < PER; e++) { kf[e] = lane_ok ? to_f<T>(kr[e]) : 0.f; vf[e] = lane_ok ? to_f<T>(vr[e]) : 0.f; }
#pragma unroll
    for (int g = 0; g < GMAX; g++) {
      if (g >= G) break;
      float s = 0.f;
#pragma unroll
      for (int e = 0; e < PER; e++) s = fmaf(q[g][e], kf[e], s);
      s = warp_sum(s) * scale;
      const float mn = fmaxf(m[g], s);
      const float a = __expf(m[g] - mn), p = __expf(s - mn);   // m = -inf on the first key: a = 0
      l[g] = l[g] * a + p;
#pragma unroll
      for (int e = 0; e < PER; e++) o[g][e] = o[g][e] * a + p * vf[e];
      m[g] = mn;
    }
  }
  // combine the four warps (fixed order)
  __shared__ float sm_m[4][GMAX], sm_l[4][GMAX];
  __shared__ float sm_o[4][GMAX][32 * PER];
#pragma unroll
  for (int g = 0; g < GMAX; g++) {
    if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
#pragma unroll
    for (int e = 0; e < PER; e++) sm_o[warp][g][lane * PER + e] = o[g][e];
  }
  __syncthreads();
  // thread t < 32*PER... each thread of the block finalises channels strided by 128
  for (int g = 0; g < G; g++) {
    float M = -INFINITY;
    for (int w = 0; w < 4; w++) M = fmaxf(M, sm_m[w][g]);
    float Lsum = 0.f;
    float wgt[4];
    for (int w = 0; w < 4; w++) { wgt[w] = sm_m[w][g] == -INFINITY ? 0.f : __expf(sm_m[w][g] - M); Lsum += sm_l[w][g] * wgt[w]; }
    float* dst = part + ((((long long)b * H + kvh * G + g) * splits + sp) * (hd + 2));
    if (threadIdx.x == 0) { dst[0] = M; dst[1] = Lsum; }
    for (int c = threadIdx.x; c < hd; c += 128) {
      float acc = 0.f;
      for (int w = 0; w < 4; w++) acc += sm_o[w][g][c] * wgt[w];
      dst[2 + c] = acc;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) k_decode_attn_combine(const float* __restrict__ part, int splits, int H, int hd,
                                                             T* __restrict__ out, long long ldo) {
  const int h = blockIdx.x, b = blockIdx.y;
  const float* p = part + ((long long)b * H + h) * splits * (hd + 2);
  float M = -INFINITY;
  for (int s = 0; s < splits; s++) M = fmaxf(M, p[(long long)s * (hd + 2)]);
  float L = 0.f;
  for (int s = 0; s < splits; s++) {
    const float ms = p[(long long)s * (hd + 2)];
    L += ms == -INFINITY ? 0.f : p[(long long)s * (hd + 2) + 1] * __expf(ms - M);
  }
  for (int c = threadIdx.x; c < hd; c += 128) {
    float acc = 0.f;
    for (int s = 0; s < splits; s++) {
      const float ms = p[(long long)s * (hd + 2)];
      if (ms != -INFINITY) acc += p[(long long)s * (hd + 2) + 2 + c] * __expf(ms - M);
    }
    out[(long long)b * ldo + (long long)h * hd + c] = from_f<T>(acc / L);
  }
}

// ---- weight-streaming product for a few rows ----------------------------------------------------------------------
// Y[M][out] = epilogue(X[M][in] W[in][ldw]) for M <= 8 rows, W in bf16 with `out` contiguous.  Every weight is read
// exactly once with 16-byte loads; a thread owns 8 output columns and one range of `in`, so the grid has
// out/8 x splits threads in flight.  Partials are summed in split order by k_rows_reduce (fixed order).
constexpr int RM = 8, KCH = 32;
__global__ void __launch_bounds__(128) k_rows_partial(const bf16* __restrict__ X, long long ldx, const bf16* __restrict__ W,
                                                      long long ldw, int M, int in, int out, float* __restrict__ part) {
  __shared__ float xs[RM][KCH];
  const int col0 = (blockIdx.x * 128 + threadIdx.x) * 8;
  const int k0 = blockIdx.y * KCH;
  const int kn = min(KCH, in - k0);
  for (int i = threadIdx.x; i < RM * KCH; i += 128) {
    const int m = i / KCH, k = i % KCH;
    xs[m][k] = (m < M && k < kn) ? __bfloat162float(X[(long long)m * ldx + k0 + k]) : 0.f;
  }
  __syncthreads();
  if (col0 >= out) return;
  float acc[RM][8];
#pragma unroll
  for (int m = 0; m < RM; m++)
#pragma unroll
    for (int j = 0; j < 8; j++) acc[m][j] = 0.f;
  const bf16* wp = W + (long long)k0 * ldw + col0;
#pragma unroll 4
  for (int k = 0; k < kn; k++) {
    const uint4 wv = *reinterpret_cast<const uint4*>(wp + (long long)k * ldw);
    const bf16* wh = reinterpret_cast<const bf16*>(&wv);
    float wf[8];
#pragma unroll
    for (int j = 0; j < 8; j++) wf[j] = __bfloat162float(wh[j]);
#pragma unroll
    for (int m = 0; m < RM; m++) {
      const float xv = xs[m][k];
#pragma unroll
      for (int j = 0; j < 8; j++) acc[m][j] = fmaf(xv, wf[j], acc[m][j]);
    }
  }
  float* dst = part + ((long long)blockIdx.y * RM) * out + col0;
#pragma unroll
  for (int m = 0; m < RM; m++) {
    if (m >= M) break;
    *reinterpret_cast<float4*>(dst + (long long)m * out) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
    *reinterpret_cast<float4*>(dst + (long long)m * out + 4) = make_float4(acc[m][4], acc[m][5], acc[m][6], acc[m][7]);
  }
}
// epi: EPI_STORE, EPI_RESID (aux may alias C), EPI_RELU2 write bf16; EPI_F32 writes fp32 (softcapped when softcap != 0)
__global__ void __launch_bounds__(256) k_rows_reduce(const float* __restrict__ part, int splits, int M, int out, int n_valid,
                                                     int epi, const bf16* aux, long long ldaux, void* C, long long ldc,
                                                     float softcap) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)M * n_valid) return;
  const int m = (int)(i / n_valid), n = (int)(i % n_valid);
  float acc = 0.f;
  for (int s = 0; s < splits; s++) acc += part[((long long)s * RM + m) * out + n];
  if (epi == EPI_F32) {
    if (softcap != 0.f) acc = softcap * tanhf(acc / softcap);
    reinterpret_cast<float*>(C)[(long long)m * ldc + n] = acc;
    return;
  }
  if (epi == EPI_RESID) acc += __bfloat162float(aux[(long long)m * ldaux + n]);
  if (epi == EPI_RELU2) { acc = fmaxf(acc, 0.f); acc *= acc; }
  reinterpret_cast<bf16*>(C)[(long long)m * ldc + n] = __float2bfloat16_rn(acc);
}

}  // namespace

// Y = epilogue(X W) for the few rows of a decode step.  bf16 with aligned operands takes the weight-streaming
// kernel; anything else the general GEMM.  n_valid <= out: only the first n_valid columns are written (logits).
template <typename T>
static int rows_product(femto_kv_cache* c, const void* X, int in, const void* W, long long ldw, int out, int n_valid, int M,
                        int epi, const void* aux, void* C, long long ldc, float softcap, cudaStream_t s) {
  femto_handle* h = c->h;
  const int splits = cdiv(in, KCH);
  const bool fast = sizeof(T) == 2 && M <= RM && (ldw & 7) == 0 && (out & 7) == 0 && aligned16(W) &&
                    (size_t)splits * RM * out <= c->part_floats;
  if (fast) {
    k_rows_partial<<<dim3(cdiv(out, 8 * 128), splits), 128, 0, s>>>((const bf16*)X, in, (const bf16*)W, ldw, M, in, out, c->part);
    KERNEL_CHECK();
    k_rows_reduce<<<cdiv((long long)M * n_valid, 256), 256, 0, s>>>(c->part, splits, M, out, n_valid, epi, (const bf16*)aux, ldc,
                                                                  C, ldc, softcap);
    KERNEL_CHECK();
    return 0;
  }
  GemmArgs g;
  g.ws = h->gemm_ws; g.ws_bytes = h->gemm_ws_bytes; g.status = h->status;
  g.A = X; g.lda = in; g.a_kmajor = true; g.B = W; g.ldb = ldw; g.b_kmajor = false;
  g.C = C; g.ldc = ldc; g.M = M; g.N = n_valid; g.K = in; g.epi = epi; g.aux = aux; g.ldaux = ldc; g.beta = 0.f;
  FEMTO_TRY(gemm<T>(g, s));
  if (epi == EPI_F32 && softcap != 0.f) FEMTO_TRY(softcap_inplace((float*)C, (long long)M * ldc, s));
  return 0;
}

template <typename T>
static int decode_attention(femto_kv_cache* c, int layer, const T* qkv, long long ldq, T* out, long long ldo, int B, int tq,
                            int window_left, const int* docs, cudaStream_t s) {
  femto_handle* h = c->h;
  const int G = h->H / h->Hkv, per = cdiv(h->hd, 32);
  if (G > 8 || per > 8 || h->hd % (per <= 4 ? 4 : 8) != 0)
    return femto_fail(FEMTO_ERR_UNSUPPORTED, "decode attention: group of %d heads / head_dim %d not supported", G, h->hd);
  const int nkeys_max = std::min(tq + 1, window_left + 1);
  int splits = std::max(1, std::min(MAX_SPLITS, cdiv(nkeys_max, 64)));
  if ((size_t)B * h->H * splits * (h->hd + 2) > c->part_floats) splits = 1;
  dim3 grid(h->Hkv, B, splits);
#define LAUNCH(PER, GM) k_decode_attn<T, PER, GM><<<grid, 128, 0, s>>>(qkv, ldq, (const T*)c->K[layer], (const T*)c->V[layer], \
    c->maxT, h->kv, tq, window_left, docs, h->H, h->Hkv, h->hd, c->part, splits)
  if (per <= 4 && G <= 2) LAUNCH(4, 2);
  else if (per <= 4) LAUNCH(4, 8);
  else if (G <= 2) LAUNCH(8, 2);
  else LAUNCH(8, 8);
#undef LAUNCH
  KERNEL_CHECK();
  k_decode_attn_combine<T><<<dim3(h->H, B), 128, 0, s>>>(c->part, splits, h->H, h->hd, out, ldo);
  KERNEL_CHECK();
  return 0;
}

// Called by the forward pass of a prompt (model.cu) once every block's packed QKV rows are in place.
template <typename T> int kv_cache_store_prompt(femto_kv_cache* c, int B, int Tp, cudaStream_t s) {
  femto_handle* h = c->h;
  if (B > c->maxB || Tp > c->maxT) return femto_fail(FEMTO_ERR_SHAPE, "prompt [%d][%d] exceeds the cache [%d][%d]", B, Tp, c->maxB, c->maxT);
  for (int i = 0; i < h->L; i++) {
    const long long n = (long long)B * Tp * h->kv;
    k_kv_prefill<T><<<cdiv(n, 256), 256, 0, s>>>((const T*)h->lb[i].qkv, h->dq, h->d, h->kv, (T*)c->K[i], (T*)c->V[i], c->maxT, Tp, B);
    KERNEL_CHECK();
  }
  k_take_last_rows<T><<<cdiv((long long)B * h->d, 256), 256, 0, s>>>((const T*)h->xe, Tp, h->d, B, (T*)c->xe_prev);
  KERNEL_CHECK();
  k_take_last_pos<<<cdiv(B, 128), 128, 0, s>>>(h->pos, Tp, B, c->lastpos);
  KERNEL_CHECK();
  c->B = B; c->len = Tp;
  return 0;
}
template int kv_cache_store_prompt<float>(femto_kv_cache*, int, int, cudaStream_t);
template int kv_cache_store_prompt<bf16>(femto_kv_cache*, int, int, cudaStream_t);

// logits of the last prompt position: rows (b, Tp-1) of the normalised head input through lm_head
template <typename T> int kv_cache_last_logits(femto_kv_cache* c, const T* xnf, int B, int Tp, float* logits_out, cudaStream_t s) {
  femto_handle* h = c->h;
  k_take_last_rows<T><<<cdiv((long long)B * h->d, 256), 256, 0, s>>>(xnf, Tp, h->d, B, (T*)c->xe_new);
  KERNEL_CHECK();
  // chunks of 8 rows through the weight-streaming product
  for (int b0 = 0; b0 < B; b0 += RM) {
    const int m = std::min(RM, B - b0);
    FEMTO_TRY(rows_product<T>(c, (const T*)c->xe_new + (size_t)b0 * h->d, h->d, h->sh_lm, h->Vp, h->Vp, h->V, m, EPI_F32, nullptr,
                              logits_out + (size_t)b0 * h->V, h->V, 15.f, s));
  }
  return 0;
}
template int kv_cache_last_logits<float>(femto_kv_cache*, const float*, int, int, float*, cudaStream_t);
template int kv_cache_last_logits<bf16>(femto_kv_cache*, const bf16*, int, int, float*, cudaStream_t);

template <typename T>
static int decode_t(femto_kv_cache* c, const float* theta, const int* tokens, const int* positions, int B, float* logits_out,
                    cudaStream_t s) {
  typedef Stream<T> S;
  femto_handle* h = c->h;
  const int d = h->d, dq = h->dq, kv = h->kv, H = h->H, Hkv = h->Hkv, hd = h->hd, L = h->L;
  const float eps = h->eps;
  const int t = c->len;   // row of the new token in every column's cache
  k_decode_prep<<<cdiv(B, 128), 128, 0, s>>>(tokens, positions, B, h->cfg.index_base, h->V, h->cfg.max_document_tokens, t, c->tok0,
                                             c->pos, c->doc_start, c->lastpos, h->status);
  KERNEL_CHECK();
  const int* docs = h->cfg.doc_mask ? c->doc_start : nullptr;
  FEMTO_TRY(S::embed_norm((const T*)h->sh_wte, c->tok0, (T*)c->xe_new, B, d, eps, s));
  k_smear_decode<T><<<cdiv(B, 8), 256, 0, s>>>((const T*)c->xe_new, (T*)c->xe_prev, theta + h->off_smear, theta + h->off_lam_s, B, d,
                                               (T*)h->x0);
  KERNEL_CHECK();
  // M rows at a time through the weight-streaming product (its register tile holds 8 rows)
  auto product = [&](const void* X, int in, const void* W, int out, void* Y, int epi, const void* aux) {
    for (int b0 = 0; b0 < B; b0 += RM) {
      const int m = std::min(RM, B - b0);
      FEMTO_TRY(rows_product<T>(c, (const T*)X + (size_t)b0 * in, in, W, out, out, out, m, epi,
                                aux ? (const T*)aux + (size_t)b0 * out : nullptr, (T*)Y + (size_t)b0 * out, out, 0.f, s));
    }
    return 0;
  };
  for (int i = 0; i < L; i++) {
    const LayerP& p = h->lp[i];
    LayerBuf& l = h->lb[i];
    const T* xin = i == 0 ? (const T*)h->x0 : (const T*)h->lb[i - 1].xout;
    FEMTO_TRY(S::mix_norm(xin, (const T*)h->x0, theta + p.lam_b, theta + p.lam_x0, (T*)h->xm, (T*)l.xn1, l.r1, B, d, eps, s));
    FEMTO_TRY(product(l.xn1, d, l.sh_wqkv, dq, l.qkv, EPI_STORE, nullptr));
    FEMTO_TRY(S::qkv_post((T*)l.qkv, dq, (const T*)l.xn1, d, p.ve ? theta + p.ve_gate : nullptr, p.ve ? (const T*)l.sh_ve : nullptr,
                          c->tok0, c->pos, h->sin_t, h->cos_t, B, H, Hkv, hd, eps, l.rqk, l.sv, s));
    k_kv_append<T><<<cdiv((long long)B * kv, 256), 256, 0, s>>>((const T*)l.qkv, dq, d, kv, (T*)c->K[i], (T*)c->V[i], c->maxT, t, B);
    KERNEL_CHECK();
    FEMTO_TRY(decode_attention<T>(c, i, (const T*)l.qkv, dq, (T*)l.att, d, B, t, p.window, docs, s));
    FEMTO_TRY(product(l.att, d, l.sh_wo, d, h->xm, EPI_RESID, h->xm));
    FEMTO_TRY(S::norm((const T*)h->xm, (T*)l.xn2, l.r2, B, d, eps, s));
    FEMTO_TRY(product(l.xn2, d, l.sh_fc, 4 * d, l.a, EPI_RELU2, nullptr));
    FEMTO_TRY(product(l.a, 4 * d, l.sh_proj, d, l.xout, EPI_RESID, h->xm));
  }
  FEMTO_TRY(S::backout_norm((const T*)h->lb[L - 1].xout, (const T*)h->lb[h->backout].xout, theta + h->off_lam_y, nullptr,
                            (T*)h->xnf, h->rf, B, d, eps, s));
  for (int b0 = 0; b0 < B; b0 += RM) {
    const int m = std::min(RM, B - b0);
    FEMTO_TRY(rows_product<T>(c, (const T*)h->xnf + (size_t)b0 * d, d, h->sh_lm, h->Vp, h->Vp, h->V, m, EPI_F32, nullptr,
                              logits_out + (size_t)b0 * h->V, h->V, 15.f, s));
  }
  c->len = t + 1;
  return 0;
}

extern "C" int32_t femto_kv_cache_create(femto_handle* h, int32_t max_batch, int32_t max_len, femto_kv_cache** out) {
  if (!h || !out || max_batch <= 0 || max_len <= 0) return femto_fail(FEMTO_ERR_ARG, "bad argument");
  *out = nullptr;
  if (max_batch > h->maxB) return femto_fail(FEMTO_ERR_SHAPE, "max_batch %d exceeds the handle's %d", max_batch, h->maxB);
  femto_kv_cache* c = new femto_kv_cache();
  c->h = h; c->maxB = max_batch; c->maxT = max_len;
  const size_t es = h->bf ? 2 : 4;
  auto al = [](size_t b) { return (b + 255) & ~(size_t)255; };
  const size_t per_layer = al(es * (size_t)max_batch * max_len * h->kv);
  // partials: decode attention [B][H][splits][hd+2]; weight-streaming product [in/32][8][out] for the widest product
  const size_t widest = std::max<size_t>({(size_t)cdiv(h->d, KCH) * RM * (size_t)h->Vp, (size_t)cdiv(4 * h->d, KCH) * RM * (size_t)h->d,
                                          (size_t)cdiv(h->d, KCH) * RM * (size_t)std::max(4 * h->d, h->dq)});
  c->part_floats = std::max(widest, (size_t)max_batch * h->H * MAX_SPLITS * (h->hd + 2));
  const size_t total = 2 * per_layer * h->L + 2 * al(es * (size_t)max_batch * h->d) + 4 * al(4 * (size_t)max_batch) + al(4 * c->part_floats);
  cudaError_t e = cudaMalloc(&c->mem, total);
  if (e != cudaSuccess) {
    delete c;
    return femto_fail(FEMTO_ERR_NOMEM, "cudaMalloc of %.2f GiB key/value cache failed: %s", total / 1073741824.0, cudaGetErrorString(e));
  }
  char* p = c->mem;
  c->K.resize(h->L); c->V.resize(h->L);
  for (int i = 0; i < h->L; i++) { c->K[i] = p; p += per_layer; c->V[i] = p; p += per_layer; }
  c->xe_prev = p; p += al(es * (size_t)max_batch * h->d);
  c->xe_new = p; p += al(es * (size_t)max_batch * h->d);
  c->tok0 = (int*)p; p += al(4 * (size_t)max_batch);
  c->pos = (int*)p; p += al(4 * (size_t)max_batch);
  c->doc_start = (int*)p; p += al(4 * (size_t)max_batch);
  c->lastpos = (int*)p; p += al(4 * (size_t)max_batch);
  c->part = (float*)p;
  *out = c;
  return 0;
}

extern "C" int32_t femto_kv_cache_destroy(femto_kv_cache* c) {
  if (!c) return 0;
  cudaDeviceSynchronize();
  cudaFree(c->mem);
  delete c;
  return 0;
}

extern "C" int32_t femto_kv_cache_length(femto_kv_cache* c) { return c ? c->len : FEMTO_ERR_ARG; }

extern "C" int32_t femto_prefill(femto_handle* h, femto_kv_cache* c, const float* theta, const int32_t* tokens,
                                 const int32_t* positions, int32_t B, int32_t Tp, float* logits_out, void* stream) {
  if (!h || !c || !theta || !tokens || !logits_out) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  if (c->h != h) return femto_fail(FEMTO_ERR_ARG, "the cache belongs to another handle");
  if (B <= 0 || B > c->maxB || Tp <= 0 || Tp > c->maxT) return femto_fail(FEMTO_ERR_SHAPE, "prompt [%d][%d] exceeds the cache [%d][%d]", B, Tp, c->maxB, c->maxT);
  if ((long long)B * Tp > h->maxN) return femto_fail(FEMTO_ERR_SHAPE, "prompt of %d x %d tokens exceeds the workspace (%d tokens)", B, Tp, h->maxN);
  StepExtra ex;
  ex.T = Tp; ex.cache = c; ex.last_logits = logits_out;
  return model_step(h, theta, nullptr, tokens, nullptr, positions, B, FEMTO_REDUCTION_SUM, false, false, nullptr, nullptr,
                    (cudaStream_t)stream, nullptr, nullptr, &ex);
}

extern "C" int32_t femto_decode_step(femto_handle* h, femto_kv_cache* c, const float* theta, const int32_t* tokens,
                                     const int32_t* positions, int32_t B, float* logits_out, void* stream) {
  if (!h || !c || !theta || !tokens || !logits_out) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  if (c->h != h) return femto_fail(FEMTO_ERR_ARG, "the cache belongs to another handle");
  if (c->len <= 0) return femto_fail(FEMTO_ERR_STATE, "femto_prefill must run before the first femto_decode_step");
  if (B != c->B) return femto_fail(FEMTO_ERR_SHAPE, "B=%d differs from the prompt's %d columns", B, c->B);
  if (c->len >= c->maxT) return femto_fail(FEMTO_ERR_SHAPE, "the cache is full (%d tokens per column)", c->maxT);
  if (!h->weights_valid) return femto_fail(FEMTO_ERR_STATE, "call femto_refresh_weights before the first step");
  return h->bf ? decode_t<bf16>(c, theta, tokens, positions, B, logits_out, (cudaStream_t)stream)
               : decode_t<float>(c, theta, tokens, positions, B, logits_out, (cudaStream_t)stream);
}
