// HBM-streaming kernels of the GPT step: one warp owns one token row (or one (token, head)
// slice), 16-byte vector loads/stores when the row length allows, fp32 statistics.
// Reference arithmetic: norm src/gpt.jl:16-20 (reverse ext/FemtoChatMooncakeExt.jl:248-255),
// smear src/gpt.jl:118-122,139-140 (reverse ext/FemtoChatMooncakeExt.jl:57-73), residual mixes
// src/gpt.jl:148,160-162, RoPE src/gpt.jl:55-77 (reverse ext/FemtoChatEnzymeExt.jl:168-169),
// QK-norm src/gpt.jl:105-106, value-embedding gate src/gpt.jl:95-99.
#include "streaming.cuh"

#include <algorithm>

namespace {

constexpr int WPB = 8;  // warps (rows) per block
#define ROW_SETUP()                                                      \
  const int lane = threadIdx.x & 31;                                     \
  const long long row = (long long)blockIdx.x * WPB + (threadIdx.x >> 5); \
  if (row >= N) return;

#define DISPATCH_V(cond, ...)                \
  if (cond) {                                \
    constexpr int V = VecN<T>::n;            \
    __VA_ARGS__                              \
  } else {                                   \
    constexpr int V = 1;                     \
    __VA_ARGS__                              \
  }

__global__ void k_prep_tokens(const int* tokens, const int* targets, const int* positions, int n, int Tlen,
                              int base, int vocab, int maxdoc, int* tok0, int* tgt0, int* pos, int* doc_start,
                              unsigned int* status) {
  pdl_trigger();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int t = i % Tlen;
  int tk = tokens[i] - base;
  if (tk < 0 || tk >= vocab) { atomicOr(status, ST_BAD_TOKEN); tk = min(max(tk, 0), vocab - 1); }
  tok0[i] = tk;
  int tg = targets ? targets[i] : -1;
  if (tg != -1) {
    tg -= base;
    if (tg < 0 || tg >= vocab) { atomicOr(status, ST_BAD_TOKEN); tg = -1; }
  }
  tgt0[i] = tg;
  int p = positions ? positions[i] : t;
  if (p < 0 || p >= maxdoc) { atomicOr(status, ST_BAD_TOKEN); p = min(max(p, 0), maxdoc - 1); }
  pos[i] = p;
  doc_start[i] = max(0, t - p);
}

template <typename T, int V>
__global__ void __launch_bounds__(256) k_embed_norm(const T* __restrict__ table, const int* __restrict__ tok0,
                                                    T* __restrict__ xe, int N, int D, float eps) {
  pdl_trigger();
  ROW_SETUP();
  const T* src = table + (long long)tok0[row] * D;
  float ss = 0.f;
  for (int c = lane * V; c < D; c += 32 * V) {
    float f[V];
    load_vec<T, V>(src + c, f);
#pragma unroll
    for (int i = 0; i < V; i++) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / D + eps);
  T* dst = xe + row * D;
  for (int c = lane * V; c < D; c += 32 * V) {
    float f[V];
    load_vec<T, V>(src + c, f);
#pragma unroll
    for (int i = 0; i < V; i++) f[i] *= inv;
    store_vec<T, V>(dst + c, f);
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(256) k_smear(const T* __restrict__ xe, const float* __restrict__ w_s,
                                               const float* __restrict__ lam_s, int N, int Tlen, int D,
                                               float* __restrict__ sg, T* __restrict__ x0) {
  pdl_trigger();
  ROW_SETUP();
  const int t = (int)(row % Tlen);
  const T* cur = xe + row * D;
  float gate = 0.f;
  if (t > 0) {
    float pre = lane < 24 ? to_f<T>(cur[lane]) * w_s[lane] : 0.f;
    pre = warp_sum(pre);
    float sig = 1.f / (1.f + expf(-pre));
    if (lane == 0) sg[row] = sig;
    gate = lam_s[0] * sig;
  } else if (lane == 0) {
    sg[row] = 0.f;
  }
  const T* prev = cur - D;
  T* dst = x0 + row * D;
  for (int c = lane * V; c < D; c += 32 * V) {
    float f[V];
    load_vec<T, V>(cur + c, f);
    if (t > 0) {
      float p[V];
      load_vec<T, V>(prev + c, p);
#pragma unroll
      for (int i = 0; i < V; i++) f[i] += gate * p[i];
    }
    store_vec<T, V>(dst + c, f);
  }
}

// xm = lam_b*xin + lam_x0*x0 (rounded to T), xn = norm(xm), r = sqrt(mean(xm^2)+eps)
template <typename T, int V>
__global__ void __launch_bounds__(256) k_mix_norm(const T* __restrict__ xin, const T* __restrict__ x0,
                                                  const float* __restrict__ lam_b, const float* __restrict__ lam_x0,
                                                  T* __restrict__ xm, T* __restrict__ xn, float* __restrict__ r,
                                                  int N, int D, float eps) {
  pdl_trigger();
  ROW_SETUP();
  const float lb = lam_b[0], l0 = lam_x0[0];
  const T* a = xin + row * D;
  const T* b = x0 + row * D;
  T* m = xm + row * D;
  float ss = 0.f;
  for (int c = lane * V; c < D; c += 32 * V) {
    float f[V], g[V];
    load_vec<T, V>(a + c, f);
    load_vec<T, V>(b + c, g);
#pragma unroll
    for (int i = 0; i < V; i++) {
      f[i] = round_to<T>(lb * f[i] + l0 * g[i]);
      ss += f[i] * f[i];
    }
    store_vec<T, V>(m + c, f);
  }
  ss = warp_sum(ss);
  const float rr = sqrtf(ss / D + eps);
  if (lane == 0) r[row] = rr;
  const float inv = 1.f / rr;
  T* o = xn + row * D;
  for (int c = lane * V; c < D; c += 32 * V) {
    float f[V], g[V];
    load_vec<T, V>(a + c, f);
    load_vec<T, V>(b + c, g);
#pragma unroll
    for (int i = 0; i < V; i++) f[i] = round_to<T>(lb * f[i] + l0 * g[i]) * inv;
    store_vec<T, V>(o + c, f);
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(256) k_norm(const T* __restrict__ x, T* __restrict__ xn, float* __restrict__ r,
                                              int N, int D, float eps) {
  pdl_trigger();
  ROW_SETUP();
  const T* a = x + row * D;
  float ss = 0.f;
  for (int c = lane * V; c < D; c += 32 * V) {
    float f[V];
    load_vec<T, V>(a + c, f);
#pragma unroll
    for (int i = 0; i < V; i++) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  const float rr = sqrtf(ss / D + eps);
  if (lane == 0) r[row] = rr;
  const float inv = 1.f / rr;
  T* o = xn + row * D;
  for (int c = lane * V; c < D; c += 32 * V) {
    float f[V];
    load_vec<T, V>(a + c, f);
#pragma unroll
    for (int i = 0; i < V; i++) f[i] *= inv;
    store_vec<T, V>(o + c, f);
  }
}

// xf = xl - lam_y*xb (rounded to T), xnf = norm(xf)
template <typename T, int V>
__global__ void __launch_bounds__(256) k_backout_norm(const T* __restrict__ xl, const T* __restrict__ xb,
                                                      const float* __restrict__ lam_y, T* __restrict__ xnf,
                                                      float* __restrict__ rf, int N, int D, float eps) {
  pdl_trigger();
  ROW_SETUP();
  const float ly = lam_y[0];
  const T* a = xl + row * D;
  const T* b = xb + row * D;
  float ss = 0.f;
  for (int c = lane * V; c < D; c += 32 * V) {
    float f[V], g[V];
    load_vec<T, V>(a + c, f);
    load_vec<T, V>(b + c, g);
#pragma unroll
    for (int i = 0; i < V; i++) {
      float v = round_to<T>(f[i] - ly * g[i]);
      ss += v * v;
    }
  }
  ss = warp_sum(ss);
  const float rr = sqrtf(ss / D + eps);
  if (lane == 0) rf[row] = rr;
  const float inv = 1.f / rr;
  T* o = xnf + row * D;
  for (int c = lane * V; c < D; c += 32 * V) {
    float f[V], g[V];
    load_vec<T, V>(a + c, f);
    load_vec<T, V>(b + c, g);
#pragma unroll
    for (int i = 0; i < V; i++) f[i] = round_to<T>(f[i] - ly * g[i]) * inv;
    store_vec<T, V>(o + c, f);
  }
}

// One warp per (token, slot): slots [0,H) = query heads, [H,H+Hkv) = key heads, then value heads.
template <typename T>
__global__ void __launch_bounds__(256) k_qkv_post(T* __restrict__ qkv, long long ldq, const T* __restrict__ xn1,
                                                  int D, const float* __restrict__ ve_gate,
                                                  const T* __restrict__ ve_table, const int* __restrict__ tok0,
                                                  const int* __restrict__ pos, const float* __restrict__ sin_t,
                                                  const float* __restrict__ cos_t, long long N, int H, int Hkv,
                                                  int hd, float eps, float* __restrict__ rqk,
                                                  float* __restrict__ sv) {
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int nslot = H + 2 * Hkv;
  const long long w = (long long)blockIdx.x * WPB + (threadIdx.x >> 5);
  if (w >= N * nslot) return;
  const long long n = w / nslot;
  const int slot = (int)(w % nslot);
  T* base = qkv + n * ldq + (long long)slot * hd;
  const int half = hd / 2;
  if (slot < H + Hkv) {
    const float* sn = sin_t + (long long)pos[n] * half;
    const float* cs = cos_t + (long long)pos[n] * half;
    float ss = 0.f;
    for (int p = lane; p < half; p += 32) {
      float x1 = to_f<T>(base[p]), x2 = to_f<T>(base[p + half]);
      float c = round_to<T>(cs[p]), s = round_to<T>(sn[p]);
      float y1 = round_to<T>(x1 * c + x2 * s), y2 = round_to<T>(-x1 * s + x2 * c);
      ss += y1 * y1 + y2 * y2;
    }
    ss = warp_sum(ss);
    const float rr = sqrtf(ss / hd + eps);
    if (lane == 0) rqk[n * (H + Hkv) + slot] = rr;
    const float g = 1.2f / rr;
    for (int p = lane; p < half; p += 32) {
      float x1 = to_f<T>(base[p]), x2 = to_f<T>(base[p + half]);
      float c = round_to<T>(cs[p]), s = round_to<T>(sn[p]);
      float y1 = round_to<T>(x1 * c + x2 * s), y2 = round_to<T>(-x1 * s + x2 * c);
      base[p] = from_f<T>(y1 * g);
      base[p + half] = from_f<T>(y2 * g);
    }
  } else if (ve_table != nullptr) {
    const int kvh = slot - H - Hkv;
    // gate = 3*sigmoid(sum_j xn1[n][j] * Wg[j][kvh]), j < 12
    float pre = lane < 12 ? to_f<T>(xn1[n * D + lane]) * ve_gate[lane * Hkv + kvh] : 0.f;
    pre = warp_sum(pre);
    const float sig = 1.f / (1.f + expf(-pre));
    if (lane == 0) sv[n * Hkv + kvh] = sig;
    const T* ve = ve_table + (long long)tok0[n] * (Hkv * hd) + (long long)kvh * hd;
    for (int d = lane; d < hd; d += 32) base[d] = from_f<T>(to_f<T>(base[d]) + 3.f * sig * to_f<T>(ve[d]));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) k_qkv_post_bwd(T* __restrict__ dqkv, const T* __restrict__ qkv,
                                                      long long ldq, const T* __restrict__ ve_table,
                                                      const int* __restrict__ tok0, const int* __restrict__ pos,
                                                      const float* __restrict__ sin_t,
                                                      const float* __restrict__ cos_t, long long N, int H, int Hkv,
                                                      int hd, const float* __restrict__ rqk,
                                                      const float* __restrict__ sv, T* __restrict__ dve,
                                                      float* __restrict__ dpre) {
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int nslot = H + 2 * Hkv;
  const long long w = (long long)blockIdx.x * WPB + (threadIdx.x >> 5);
  if (w >= N * nslot) return;
  const long long n = w / nslot;
  const int slot = (int)(w % nslot);
  T* g = dqkv + n * ldq + (long long)slot * hd;
  const T* y = qkv + n * ldq + (long long)slot * hd;
  const int half = hd / 2;
  if (slot < H + Hkv) {
    // forward: out = 1.2 * yr / r, yr = rope(x).  reverse of the norm with yhat = out/1.2:
    // dyr = (gq - yhat * mean(gq*yhat)) / r with gq = 1.2*dout; then the transposed rotation.
    float dot = 0.f;
    for (int d = lane; d < hd; d += 32) dot += to_f<T>(g[d]) * to_f<T>(y[d]);
    dot = warp_sum(dot) / hd;  // = mean(gq*yhat) since (1.2 g)(y/1.2) = g*y
    const float rr = rqk[n * (H + Hkv) + slot];
    const float* sn = sin_t + (long long)pos[n] * half;
    const float* cs = cos_t + (long long)pos[n] * half;
    for (int p = lane; p < half; p += 32) {
      float g1 = 1.2f * to_f<T>(g[p]), g2 = 1.2f * to_f<T>(g[p + half]);
      float h1 = to_f<T>(y[p]) * (1.f / 1.2f), h2 = to_f<T>(y[p + half]) * (1.f / 1.2f);
      float d1 = (g1 - h1 * dot) / rr, d2 = (g2 - h2 * dot) / rr;
      float c = round_to<T>(cs[p]), s = round_to<T>(sn[p]);
      g[p] = from_f<T>(d1 * c - d2 * s);
      g[p + half] = from_f<T>(d1 * s + d2 * c);
    }
  } else if (ve_table != nullptr) {
    const int kvh = slot - H - Hkv;
    const T* ve = ve_table + (long long)tok0[n] * (Hkv * hd) + (long long)kvh * hd;
    const float sig = sv[n * Hkv + kvh];
    float dg = 0.f;
    T* out = dve + n * (Hkv * hd) + (long long)kvh * hd;
    for (int d = lane; d < hd; d += 32) {
      float dv = to_f<T>(g[d]);
      dg += dv * to_f<T>(ve[d]);
      out[d] = from_f<T>(3.f * sig * dv);
    }
    dg = warp_sum(dg);
    if (lane == 0) dpre[n * Hkv + kvh] = dg * 3.f * sig * (1.f - sig);
  }
}


// head_dim 128 specialisation: 8 lanes per (token, slot), 16 channels per lane (8 RoPE pairs), one pass
// with the rotated values kept in registers and 16-byte (bf16) / 32-byte (fp32) accesses: with fewer bytes
// per thread the kernel was bound by loads in flight, not by HBM.
__device__ __forceinline__ float oct_sum(float v) {
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
  if constexpr (sizeof(T) == 4) {
    const float4 u = *reinterpret_cast<const float4*>(p), w = *reinterpret_cast<const float4*>(p + 4);
    f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w; f[4] = w.x; f[5] = w.y; f[6] = w.z; f[7] = w.w;
  } else {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const bf16* h = reinterpret_cast<const bf16*>(&v);
#pragma unroll
    for (int i = 0; i < 8; i++) f[i] = __bfloat162float(h[i]);
  }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&f)[8]) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  } else {
    uint4 v;
    bf16* h = reinterpret_cast<bf16*>(&v);
#pragma unroll
    for (int i = 0; i < 8; i++) h[i] = __float2bfloat16_rn(f[i]);
    *reinterpret_cast<uint4*>(p) = v;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) k_qkv_post_128(T* __restrict__ qkv, long long ldq, const T* __restrict__ xn1, int D,
                                                      const float* __restrict__ ve_gate, const T* __restrict__ ve_table,
                                                      const int* __restrict__ tok0, const int* __restrict__ pos,
                                                      const float* __restrict__ sin_t, const float* __restrict__ cos_t,
                                                      long long N, int H, int Hkv, float eps, float* __restrict__ rqk,
                                                      float* __restrict__ sv) {
  pdl_trigger();
  constexpr int hd = 128, half = 64;
  const int sub = threadIdx.x & 7;
  const int nslot = H + 2 * Hkv;
  const long long w0 = (long long)blockIdx.x * 32 + (threadIdx.x >> 3);
  const bool live = w0 < N * nslot;  // surplus groups recompute the last slot but never store
  const long long w = live ? w0 : N * nslot - 1;
  const long long n = w / nslot;
  const int slot = (int)(w % nslot);
  T* base = qkv + n * ldq + (long long)slot * hd;
  if (slot < H + Hkv) {
    float x1[8], x2[8], cs[8], sn[8];
    const long long tp = (long long)pos[n] * half + sub * 8;
    load8<T>(base + sub * 8, x1);
    load8<T>(base + half + sub * 8, x2);
    load8<float>(cos_t + tp, cs);
    load8<float>(sin_t + tp, sn);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const float c = round_to<T>(cs[i]), s = round_to<T>(sn[i]);
      const float y1 = round_to<T>(x1[i] * c + x2[i] * s), y2 = round_to<T>(-x1[i] * s + x2[i] * c);
      x1[i] = y1; x2[i] = y2;
      ss += y1 * y1 + y2 * y2;
    }
    ss = oct_sum(ss);
    const float rr = sqrtf(ss / hd + eps);
    if (live && sub == 0) rqk[n * (H + Hkv) + slot] = rr;
    const float g = 1.2f / rr;
#pragma unroll
    for (int i = 0; i < 8; i++) { x1[i] *= g; x2[i] *= g; }
    if (live) { store8<T>(base + sub * 8, x1); store8<T>(base + half + sub * 8, x2); }
  } else if (ve_table != nullptr) {
    const int kvh = slot - H - Hkv;
    // gate input: the first 12 channels of the normed block input, two per lane for lanes 0-3
    float pre = to_f<T>(xn1[n * D + sub]) * ve_gate[sub * Hkv + kvh];
    if (sub < 4) pre += to_f<T>(xn1[n * D + sub + 8]) * ve_gate[(sub + 8) * Hkv + kvh];
    pre = oct_sum(pre);
    const float sig = 1.f / (1.f + expf(-pre));
    if (live && sub == 0) sv[n * Hkv + kvh] = sig;
    const T* ve = ve_table + (long long)tok0[n] * (Hkv * hd) + (long long)kvh * hd + sub * 16;
    float a[8], b[8], e0[8], e1[8];
    load8<T>(base + sub * 16, a); load8<T>(base + sub * 16 + 8, b);
    load8<T>(ve, e0); load8<T>(ve + 8, e1);
#pragma unroll
    for (int i = 0; i < 8; i++) { a[i] += 3.f * sig * e0[i]; b[i] += 3.f * sig * e1[i]; }
    if (live) { store8<T>(base + sub * 16, a); store8<T>(base + sub * 16 + 8, b); }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) k_qkv_post_bwd_128(T* __restrict__ dqkv, const T* __restrict__ qkv, long long ldq,
                                                          const T* __restrict__ ve_table, const int* __restrict__ tok0,
                                                          const int* __restrict__ pos, const float* __restrict__ sin_t,
                                                          const float* __restrict__ cos_t, long long N, int H, int Hkv,
                                                          const float* __restrict__ rqk, const float* __restrict__ sv,
                                                          T* __restrict__ dve, float* __restrict__ dpre) {
  pdl_trigger();
  constexpr int hd = 128, half = 64;
  const int sub = threadIdx.x & 7;
  const int nslot = H + 2 * Hkv;
  const long long w0 = (long long)blockIdx.x * 32 + (threadIdx.x >> 3);
  const bool live = w0 < N * nslot;  // surplus groups recompute the last slot but never store
  const long long w = live ? w0 : N * nslot - 1;
  const long long n = w / nslot;
  const int slot = (int)(w % nslot);
  T* g = dqkv + n * ldq + (long long)slot * hd;
  const T* y = qkv + n * ldq + (long long)slot * hd;
  if (slot < H + Hkv) {
    float g1[8], g2[8], y1[8], y2[8], cs[8], sn[8];
    const long long tp = (long long)pos[n] * half + sub * 8;
    const float rq = rqk[n * (H + Hkv) + slot];
    load8<T>(g + sub * 8, g1); load8<T>(g + half + sub * 8, g2);
    load8<T>(y + sub * 8, y1); load8<T>(y + half + sub * 8, y2);
    load8<float>(cos_t + tp, cs);
    load8<float>(sin_t + tp, sn);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) dot += g1[i] * y1[i] + g2[i] * y2[i];
    dot = oct_sum(dot) / hd;
    const float inv = 1.f / rq;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const float d1 = (1.2f * g1[i] - y1[i] * (1.f / 1.2f) * dot) * inv, d2 = (1.2f * g2[i] - y2[i] * (1.f / 1.2f) * dot) * inv;
      const float c = round_to<T>(cs[i]), s = round_to<T>(sn[i]);
      g1[i] = d1 * c - d2 * s;
      g2[i] = d1 * s + d2 * c;
    }
    if (live) { store8<T>(g + sub * 8, g1); store8<T>(g + half + sub * 8, g2); }
  } else if (ve_table != nullptr) {
    const int kvh = slot - H - Hkv;
    const T* ve = ve_table + (long long)tok0[n] * (Hkv * hd) + (long long)kvh * hd + sub * 16;
    const float sig = sv[n * Hkv + kvh];
    float a[8], b[8], e0[8], e1[8];
    load8<T>(g + sub * 16, a); load8<T>(g + sub * 16 + 8, b);
    load8<T>(ve, e0); load8<T>(ve + 8, e1);
    float dg = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) { dg += a[i] * e0[i] + b[i] * e1[i]; a[i] *= 3.f * sig; b[i] *= 3.f * sig; }
    T* out = dve + n * (Hkv * hd) + (long long)kvh * hd + sub * 16;
    if (live) { store8<T>(out, a); store8<T>(out + 8, b); }
    dg = oct_sum(dg);
    if (live && sub == 0) dpre[n * Hkv + kvh] = dg * 3.f * sig * (1.f - sig);
  }
}

// dxn[n][j] += sum_h dpre[n][h] * Wg[j][h] (j < 12); partial[block][j*Hkv+h] = sum_n xn1[n][j]*dpre[n][h].
template <typename T>
__global__ void __launch_bounds__(256) k_ve_gate_bwd(const T* __restrict__ xn1, int D, const float* __restrict__ dpre,
                                                     const float* __restrict__ ve_gate, T* __restrict__ dxn, int N,
                                                     int Hkv, float* __restrict__ partial) {
  pdl_trigger();
  constexpr int CH = 256;
  __shared__ float sx[CH][12];
  extern __shared__ float sd[];  // [CH][Hkv]
  const int n0 = blockIdx.x * CH;
  const int cnt = min(CH, N - n0);
  for (int i = threadIdx.x; i < cnt * 12; i += blockDim.x) sx[i / 12][i % 12] = to_f<T>(xn1[(long long)(n0 + i / 12) * D + i % 12]);
  for (int i = threadIdx.x; i < cnt * Hkv; i += blockDim.x) sd[i] = dpre[(long long)n0 * Hkv + i];
  __syncthreads();
  for (int i = threadIdx.x; i < cnt * 12; i += blockDim.x) {
    int nn = i / 12, j = i % 12;
    float acc = 0.f;
    for (int h = 0; h < Hkv; h++) acc += sd[nn * Hkv + h] * ve_gate[j * Hkv + h];
    T* p = dxn + (long long)(n0 + nn) * D + j;
    *p = from_f<T>(to_f<T>(*p) + acc);
  }
  for (int o = threadIdx.x; o < 12 * Hkv; o += blockDim.x) {
    int j = o / Hkv, h = o % Hkv;
    float acc = 0.f;
    for (int nn = 0; nn < cnt; nn++) acc += sx[nn][j] * sd[nn * Hkv + h];
    partial[(long long)blockIdx.x * 12 * Hkv + o] = acc;
  }
}

// out = resid + (dy - y*mean(dy*y)) / r
template <typename T, int V>
__global__ void __launch_bounds__(256) k_norm_bwd_resid(const T* __restrict__ dy, const T* __restrict__ y,
                                                        const float* __restrict__ r, const T* resid,
                                                        T* out, int N, int D) {
  pdl_trigger();
  ROW_SETUP();
  const T* a = dy + row * D;
  const T* b = y + row * D;
  float dot = 0.f;
  for (int c = lane * V; c < D; c += 32 * V) {
    float f[V], g[V];
    load_vec<T, V>(a + c, f);
    load_vec<T, V>(b + c, g);
#pragma unroll
    for (int i = 0; i < V; i++) dot += f[i] * g[i];
  }
  dot = warp_sum(dot) / D;
  const float inv = 1.f / r[row];
  for (int c = lane * V; c < D; c += 32 * V) {
    float f[V], g[V], q[V];
    load_vec<T, V>(a + c, f);
    load_vec<T, V>(b + c, g);
    if (resid) load_vec<T, V>(resid + row * D + c, q);
#pragma unroll
    for (int i = 0; i < V; i++) f[i] = (resid ? q[i] : 0.f) + (f[i] - g[i] * dot) * inv;
    store_vec<T, V>(out + row * D + c, f);
  }
}

// dxm = dx_in + normbwd(dxn; xn1, r1); partial sums of dxm*xin and dxm*x0; dx <- lam_b*dxm (dx may be dx_in);
// dx0 (+)= lam_x0*dxm.  Rows are assigned to warps in a fixed pattern so the partials are
// reproducible.
template <typename T, int V>
__global__ void __launch_bounds__(256) k_mix_bwd(const T* dx_in, T* dx, const T* __restrict__ dxn,
                                                 const T* __restrict__ xn1, const float* __restrict__ r1,
                                                 const T* __restrict__ xin, const T* __restrict__ x0,
                                                 const float* __restrict__ lam_b, const float* __restrict__ lam_x0,
                                                 T* __restrict__ dx0, int first, int N, int D,
                                                 float* __restrict__ partial) {
  pdl_trigger();
  __shared__ float red[WPB][2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float lb = lam_b[0], l0 = lam_x0[0];
  float s_in = 0.f, s_0 = 0.f;
  for (long long row = (long long)blockIdx.x * WPB + warp; row < N; row += (long long)gridDim.x * WPB) {
    const T* a = dxn + row * D;
    const T* b = xn1 + row * D;
    float dot = 0.f;
    for (int c = lane * V; c < D; c += 32 * V) {
      float f[V], g[V];
      load_vec<T, V>(a + c, f);
      load_vec<T, V>(b + c, g);
#pragma unroll
      for (int i = 0; i < V; i++) dot += f[i] * g[i];
    }
    dot = warp_sum(dot) / D;
    const float inv = 1.f / r1[row];
    for (int c = lane * V; c < D; c += 32 * V) {
      float f[V], g[V], q[V], xi[V], xz[V], z[V];
      load_vec<T, V>(a + c, f);
      load_vec<T, V>(b + c, g);
      load_vec<T, V>(dx_in + row * D + c, q);
      load_vec<T, V>(xin + row * D + c, xi);
      load_vec<T, V>(x0 + row * D + c, xz);
      if (!first) load_vec<T, V>(dx0 + row * D + c, z);
#pragma unroll
      for (int i = 0; i < V; i++) {
        float dxm = round_to<T>(q[i] + (f[i] - g[i] * dot) * inv);
        s_in += dxm * xi[i];
        s_0 += dxm * xz[i];
        q[i] = lb * dxm;
        z[i] = (first ? 0.f : z[i]) + l0 * dxm;
      }
      store_vec<T, V>(dx + row * D + c, q);
      store_vec<T, V>(dx0 + row * D + c, z);
    }
  }
  s_in = warp_sum(s_in);
  s_0 = warp_sum(s_0);
  if (lane == 0) { red[warp][0] = s_in; red[warp][1] = s_0; }
  __syncthreads();
  if (threadIdx.x < 2) {
    float acc = 0.f;
    for (int w = 0; w < WPB; w++) acc += red[w][threadIdx.x];
    partial[blockIdx.x * 2 + threadIdx.x] = acc;
  }
}

// dxf = normbwd(dxnf; xnf, rf); partial[block] = -sum(dxf*xb)
template <typename T, int V>
__global__ void __launch_bounds__(256) k_head_bwd(const T* __restrict__ dxnf, const T* __restrict__ xnf,
                                                  const float* __restrict__ rf, const T* __restrict__ xb,
                                                  T* __restrict__ dxf, int N, int D, float* __restrict__ partial) {
  pdl_trigger();
  __shared__ float red[WPB];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float sb = 0.f;
  for (long long row = (long long)blockIdx.x * WPB + warp; row < N; row += (long long)gridDim.x * WPB) {
    const T* a = dxnf + row * D;
    const T* b = xnf + row * D;
    float dot = 0.f;
    for (int c = lane * V; c < D; c += 32 * V) {
      float f[V], g[V];
      load_vec<T, V>(a + c, f);
      load_vec<T, V>(b + c, g);
#pragma unroll
      for (int i = 0; i < V; i++) dot += f[i] * g[i];
    }
    dot = warp_sum(dot) / D;
    const float inv = 1.f / rf[row];
    for (int c = lane * V; c < D; c += 32 * V) {
      float f[V], g[V], xbv[V];
      load_vec<T, V>(a + c, f);
      load_vec<T, V>(b + c, g);
      load_vec<T, V>(xb + row * D + c, xbv);
#pragma unroll
      for (int i = 0; i < V; i++) {
        f[i] = round_to<T>((f[i] - g[i] * dot) * inv);
        sb -= f[i] * xbv[i];
      }
      store_vec<T, V>(dxf + row * D + c, f);
    }
  }
  sb = warp_sum(sb);
  if (lane == 0) red[warp] = sb;
  __syncthreads();
  if (threadIdx.x == 0) {
    float acc = 0.f;
    for (int w = 0; w < WPB; w++) acc += red[w];
    partial[blockIdx.x] = acc;
  }
}

template <typename T>
__global__ void k_axpy(T* __restrict__ y, const T* __restrict__ x, const float* a_dev, float a_mul, long long n) {
  pdl_trigger();
  const float a = (a_dev ? a_dev[0] : 1.f) * a_mul;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    y[i] = from_f<T>(to_f<T>(y[i]) + a * to_f<T>(x[i]));
}
// the same on 16-byte vectors (n a multiple of V, both pointers 16-byte aligned)
template <typename T, int V>
__global__ void __launch_bounds__(256) k_axpy_vec(T* __restrict__ y, const T* __restrict__ x, const float* a_dev, float a_mul,
                                                  long long nvec) {
  pdl_trigger();
  const float a = (a_dev ? a_dev[0] : 1.f) * a_mul;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float f[V], g[V];
    load_vec<T, V>(y + i * V, f);
    load_vec<T, V>(x + i * V, g);
#pragma unroll
    for (int e = 0; e < V; e++) f[e] = round_to<T>(f[e] + a * g[e]);
    store_vec<T, V>(y + i * V, f);
  }
}

// Row n (t >= 1): dgate = dot(dx0[n], xe[n-1]); dpre[n] = dgate*lam_s*sg*(1-sg);
// partial[block][j] = sum xe[n][j]*dpre[n] (j<24, smear gate weights), partial[block][24] = sum dgate*sg (lam_s).
template <typename T, int V>
__global__ void __launch_bounds__(256) k_smear_gate_bwd(const T* __restrict__ dx0, const T* __restrict__ xe,
                                                        const float* __restrict__ sg, const float* __restrict__ lam_s,
                                                        int N, int Tlen, int D, float* __restrict__ dpre,
                                                        float* __restrict__ partial) {
  pdl_trigger();
  __shared__ float red[WPB][25];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float ls = lam_s[0];
  float acc_l = 0.f, acc_w = 0.f;  // lane j < 24 accumulates w_s[j]
  for (long long row = (long long)blockIdx.x * WPB + warp; row < N; row += (long long)gridDim.x * WPB) {
    const int t = (int)(row % Tlen);
    if (t == 0) { if (lane == 0) dpre[row] = 0.f; continue; }
    const T* a = dx0 + row * D;
    const T* b = xe + (row - 1) * D;
    float dot = 0.f;
    for (int c = lane * V; c < D; c += 32 * V) {
      float f[V], g[V];
      load_vec<T, V>(a + c, f);
      load_vec<T, V>(b + c, g);
#pragma unroll
      for (int i = 0; i < V; i++) dot += f[i] * g[i];
    }
    dot = warp_sum(dot);
    const float sig = sg[row];
    const float dp = dot * ls * sig * (1.f - sig);
    if (lane == 0) dpre[row] = dp;
    acc_l += dot * sig;
    if (lane < 24) acc_w += to_f<T>(xe[row * D + lane]) * dp;
  }
  if (lane < 24) red[warp][lane] = acc_w;
  if (lane == 0) red[warp][24] = acc_l;
  __syncthreads();
  if (threadIdx.x < 25) {
    float acc = 0.f;
    for (int w = 0; w < WPB; w++) acc += red[w][threadIdx.x];
    partial[blockIdx.x * 25 + threadIdx.x] = acc;
  }
}

// dxe = dx0[n] + gate[n+1]*dx0[n+1] + dpre[n]*w_s (first 24 channels); dE = normbwd(dxe; xe, r(E)).
template <typename T, int V>
__global__ void __launch_bounds__(256) k_embed_bwd(const T* __restrict__ dx0, const T* __restrict__ table,
                                                   const int* __restrict__ tok0, const T* __restrict__ xe,
                                                   const float* __restrict__ sg, const float* __restrict__ dpre,
                                                   const float* __restrict__ w_s, const float* __restrict__ lam_s,
                                                   int N, int Tlen, int D, float eps, T* __restrict__ dE) {
  pdl_trigger();
  ROW_SETUP();
  const int t = (int)(row % Tlen);
  const bool has_next = t + 1 < Tlen;
  const float gnext = has_next ? lam_s[0] * sg[row + 1] : 0.f;
  const float dp = dpre[row];
  const T* src = table + (long long)tok0[row] * D;
  float ss = 0.f, dot = 0.f;
  for (int c = lane * V; c < D; c += 32 * V) {
    float e[V], f[V], nx[V], y[V];
    load_vec<T, V>(src + c, e);
    load_vec<T, V>(dx0 + row * D + c, f);
    load_vec<T, V>(xe + row * D + c, y);
    if (has_next) load_vec<T, V>(dx0 + (row + 1) * D + c, nx);
#pragma unroll
    for (int i = 0; i < V; i++) {
      ss += e[i] * e[i];
      float g = f[i] + (has_next ? gnext * nx[i] : 0.f) + ((c + i) < 24 ? dp * w_s[c + i] : 0.f);
      dot += g * y[i];
    }
  }
  ss = warp_sum(ss);
  dot = warp_sum(dot) / D;
  const float inv = rsqrtf(ss / D + eps);
  for (int c = lane * V; c < D; c += 32 * V) {
    float f[V], nx[V], y[V];
    load_vec<T, V>(dx0 + row * D + c, f);
    load_vec<T, V>(xe + row * D + c, y);
    if (has_next) load_vec<T, V>(dx0 + (row + 1) * D + c, nx);
#pragma unroll
    for (int i = 0; i < V; i++) {
      float g = f[i] + (has_next ? gnext * nx[i] : 0.f) + ((c + i) < 24 ? dp * w_s[c + i] : 0.f);
      f[i] = (g - y[i] * dot) * inv;
    }
    store_vec<T, V>(dE + row * D + c, f);
  }
}

// One block per row of fp32 logits: z = 15 tanh(l/15), lse, loss, dlogit (src/gpt.jl:12,172-194;
// src/kernels.jl:16-28; ext/FemtoChatEnzymeExt.jl:175-189).
template <typename T>
__global__ void __launch_bounds__(256) k_xent_rows(const float* __restrict__ logits, long long ldl,
                                                   const int* __restrict__ tgt0, int V, float w_host,
                                                   const float* __restrict__ w_dev, T* __restrict__ dlogit,
                                                   long long lddl,
                                                   float* __restrict__ loss_rows) {
  pdl_trigger();
  __shared__ float red[8];
  __shared__ float bc;
  const long long row = blockIdx.x;
  const float w = w_host * (w_dev ? w_dev[0] : 1.f);
  const float* l = logits + row * ldl;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float mx = -INFINITY;
  for (int v = threadIdx.x; v < V; v += 256) mx = fmaxf(mx, 15.f * tanhf(l[v] * (1.f / 15.f)));
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  if (threadIdx.x == 0) { float m = red[0]; for (int i = 1; i < 8; i++) m = fmaxf(m, red[i]); bc = m; }
  __syncthreads();
  mx = bc;
  float sum = 0.f;
  for (int v = threadIdx.x; v < V; v += 256) sum += expf(15.f * tanhf(l[v] * (1.f / 15.f)) - mx);
  sum = warp_sum(sum);
  __syncthreads();
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  if (threadIdx.x == 0) { float a = 0.f; for (int i = 0; i < 8; i++) a += red[i]; bc = a; }
  __syncthreads();
  const float lse = mx + logf(bc);
  const int tg = tgt0[row];
  if (threadIdx.x == 0) loss_rows[row] = tg >= 0 ? lse - 15.f * tanhf(l[tg] * (1.f / 15.f)) : 0.f;
  T* dl = dlogit + row * lddl;
  for (int v = threadIdx.x; v < V; v += 256) {
    float th = tanhf(l[v] * (1.f / 15.f));
    float z = 15.f * th;
    float dz = tg >= 0 ? w * (expf(z - lse) - (v == tg ? 1.f : 0.f)) : 0.f;
    dl[v] = from_f<T>(dz * (1.f - th * th));
  }
}

template <typename T> __global__ void k_cast(const float* __restrict__ src, T* __restrict__ dst, long long n) {
  pdl_trigger();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = from_f<T>(src[i]);
}
// dst [D][D+2kv] <- wq [D][D] | wk [D][kv] | wv [D][kv]
template <typename T>
__global__ void k_pack_qkv(const float* __restrict__ wq, const float* __restrict__ wk, const float* __restrict__ wv,
                           T* __restrict__ dst, int D, int kv) {
  pdl_trigger();
  const int W = D + 2 * kv;
  const long long n = (long long)D * W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    int r = (int)(i / W), c = (int)(i % W);
    float v = c < D ? wq[(long long)r * D + c] : (c < D + kv ? wk[(long long)r * kv + (c - D)] : wv[(long long)r * kv + (c - D - kv)]);
    dst[i] = from_f<T>(v);
  }
}

__global__ void __launch_bounds__(1024) k_sum_rows(const float* __restrict__ rows, int n, float* out,
                                                   const int* __restrict__ tgt0, int* n_valid_out,
                                                   float scale_by_valid) {
  pdl_trigger();
  __shared__ float red[32];
  __shared__ int redc[32];
  float acc = 0.f;
  int cnt = 0;
  // fixed assignment of rows to threads, fixed tree: reproducible
  for (int i = threadIdx.x; i < n; i += 1024) {
    acc += rows[i];
    if (tgt0 && tgt0[i] >= 0) cnt++;
  }
  acc = warp_sum(acc);
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = acc; redc[threadIdx.x >> 5] = cnt; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f;
    int c = 0;
    for (int i = 0; i < 32; i++) { a += red[i]; c += redc[i]; }
    if (scale_by_valid != 0.f) a = a / (float)c;
    *out = a;
    if (n_valid_out) *n_valid_out = c;
  }
}

// One warp per column: the lanes take every 32nd row, then a fixed shuffle tree (repeatable).  A single thread per
// column walking several hundred rows took 17 us per launch, 32 launches per step on the dependency chain.
__global__ void __launch_bounds__(256) k_reduce_partials(const float* __restrict__ partial, int nrow, int ncol,
                                                         float* out, const float* scale_dev, float scale,
                                                         int accumulate) {
  pdl_trigger();
  const int j = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (j >= ncol) return;
  float acc = 0.f;
  for (int i = lane; i < nrow; i += 32) acc += partial[(long long)i * ncol + j];
  acc = warp_sum(acc);
  if (lane == 0) {
    acc *= scale * (scale_dev ? scale_dev[0] : 1.f);
    out[j] = (accumulate ? out[j] : 0.f) + acc;
  }
}

// One warp per row: merge the row's (max, sum exp) partials into its logsumexp.
__global__ void __launch_bounds__(256) k_xent_finalize(const float2* __restrict__ stats, int ntile,
                                                       const float* __restrict__ tz, const int* __restrict__ tgt0,
                                                       int n, float* __restrict__ lse, float* __restrict__ loss_rows) {
  pdl_trigger();
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n) return;
  const float2* st = stats + (long long)row * ntile;
  float m = -INFINITY;
  for (int i = lane; i < ntile; i += 32) m = fmaxf(m, st[i].x);
  m = warp_max(m);
  float s = 0.f;
  for (int i = lane; i < ntile; i += 32) {
    const float2 v = st[i];
    s += v.y * expf(v.x - m);
  }
  s = warp_sum(s);
  if (lane == 0) {
    const float l = m + logf(s);
    lse[row] = l;
    loss_rows[row] = tgt0[row] >= 0 ? l - tz[row] : 0.f;
  }
}

// In place on a chunk of stored bf16 logits l[row][col]: d loss / d logit = w (softmax(z) - onehot) (1 - tanh^2(l/15)),
// z = 15 tanh(l/15), with the row's logsumexp from the statistics pass (src/kernels.jl:16-28;
// ext/FemtoChatEnzymeExt.jl:175-189).  Same tanh.approx / ex2 arithmetic as that pass, so softmax sums to 1 over
// the stored values.  A thread takes four 8-column groups 2048 columns apart (all four loads in flight before the
// arithmetic); rows with an ignored target become zero.
__global__ void __launch_bounds__(256) k_xent_dlogit_inplace(bf16* __restrict__ buf, long long ld,
                                                             const float* __restrict__ lse_rows,
                                                             const int* __restrict__ tgt0, int V, float w_host,
                                                             const float* __restrict__ w_dev) {
  pdl_trigger();
  const long long row = blockIdx.y;
  const int col0 = blockIdx.x * 8192 + threadIdx.x * 8;
  const int tg = tgt0[row];
  const float w = tg >= 0 ? w_host * (w_dev ? w_dev[0] : 1.f) : 0.f;
  const float lse = lse_rows[row];
  bf16* base = buf + row * ld;
  uint4 q[4];
#pragma unroll
  for (int u = 0; u < 4; u++)
    if (col0 + u * 2048 < V) q[u] = *reinterpret_cast<const uint4*>(base + col0 + u * 2048);
#pragma unroll
  for (int u = 0; u < 4; u++) {
    const int col = col0 + u * 2048;
    if (col >= V) continue;
    bf16* h = reinterpret_cast<bf16*>(&q[u]);
#pragma unroll
    for (int e = 0; e < 8; e++) {
      float t;
      asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(__bfloat162float(h[e]) * (1.f / 15.f)));
      const float z = 15.f * t;
      const float dz = w * (__expf(z - lse) - ((col + e) == tg ? 1.f : 0.f));
      h[e] = __float2bfloat16_rn(dz * (1.f - t * t));
    }
    *reinterpret_cast<uint4*>(base + col) = q[u];
  }
}

inline int row_grid(long long N) { return cdiv(N, WPB); }
inline int red_grid(long long N) { return (int)std::min<long long>(cdiv(N, WPB), 592); }

}  // namespace

template <typename T>
int Stream<T>::prep_tokens(const int* tokens, const int* targets, const int* positions, int B, int Tlen,
                           int index_base, int vocab, int maxdoc, int* tok0, int* tgt0, int* pos, int* doc_start,
                           unsigned int* status, cudaStream_t s) {
  int n = B * Tlen;
  k_prep_tokens<<<cdiv(n, 256), 256, 0, s>>>(tokens, targets, positions, n, Tlen, index_base, vocab, maxdoc, tok0,
                                             tgt0, pos, doc_start, status);
  KERNEL_CHECK();
  return 0;
}
template <typename T>
int Stream<T>::embed_norm(const T* table, const int* tok0, T* xe, int N, int D, float eps, cudaStream_t s) {
  DISPATCH_V(D % VecN<T>::n == 0, k_embed_norm<T, V><<<row_grid(N), 256, 0, s>>>(table, tok0, xe, N, D, eps);)
  KERNEL_CHECK();
  return 0;
}
template <typename T>
int Stream<T>::smear(const T* xe, const float* w_s, const float* lam_s, int N, int Tlen, int D, float* sg, T* x0,
                     cudaStream_t s) {
  if (D < 24) return femto_fail(FEMTO_ERR_SHAPE, "smear gate reads 24 channels, n_embed=%d", D);
  DISPATCH_V(D % VecN<T>::n == 0, k_smear<T, V><<<row_grid(N), 256, 0, s>>>(xe, w_s, lam_s, N, Tlen, D, sg, x0);)
  KERNEL_CHECK();
  return 0;
}
template <typename T>
int Stream<T>::mix_norm(const T* xin, const T* x0, const float* lam_b, const float* lam_x0, T* xm, T* xn, float* r,
                        int N, int D, float eps, cudaStream_t s) {
  DISPATCH_V(D % VecN<T>::n == 0, k_mix_norm<T, V><<<row_grid(N), 256, 0, s>>>(xin, x0, lam_b, lam_x0, xm, xn, r, N, D, eps);)
  KERNEL_CHECK();
  return 0;
}
template <typename T> int Stream<T>::norm(const T* x, T* xn, float* r, int N, int D, float eps, cudaStream_t s) {
  DISPATCH_V(D % VecN<T>::n == 0, k_norm<T, V><<<row_grid(N), 256, 0, s>>>(x, xn, r, N, D, eps);)
  KERNEL_CHECK();
  return 0;
}
template <typename T>
int Stream<T>::qkv_post(T* qkv, long long ldq, const T* xn1, int D, const float* ve_gate, const T* ve_table,
                        const int* tok0, const int* pos, const float* sin_t, const float* cos_t, int N, int H,
                        int Hkv, int hd, float eps, float* rqk, float* sv, cudaStream_t s) {
  long long warps = (long long)N * (H + 2 * Hkv);
  if (hd == 128 && ldq % 8 == 0 && aligned16(qkv) && (!ve_table || aligned16(ve_table)))
    k_qkv_post_128<T><<<cdiv(warps, 32), 256, 0, s>>>(qkv, ldq, xn1, D, ve_gate, ve_table, tok0, pos, sin_t, cos_t, N, H,
                                                     Hkv, eps, rqk, sv);
  else
    k_qkv_post<T><<<cdiv(warps, WPB), 256, 0, s>>>(qkv, ldq, xn1, D, ve_gate, ve_table, tok0, pos, sin_t, cos_t, N, H,
                                                  Hkv, hd, eps, rqk, sv);
  KERNEL_CHECK();
  return 0;
}
template <typename T>
int Stream<T>::qkv_post_bwd(T* dqkv, const T* qkv, long long ldq, const T* ve_table, const int* tok0,
                            const int* pos, const float* sin_t, const float* cos_t, int N, int H, int Hkv, int hd,
                            const float* rqk, const float* sv, T* dve, float* dpre, cudaStream_t s) {
  long long warps = (long long)N * (H + 2 * Hkv);
  if (hd == 128 && ldq % 8 == 0 && aligned16(qkv) && aligned16(dqkv) && (!ve_table || (aligned16(ve_table) && aligned16(dve))))
    k_qkv_post_bwd_128<T><<<cdiv(warps, 32), 256, 0, s>>>(dqkv, qkv, ldq, ve_table, tok0, pos, sin_t, cos_t, N, H, Hkv,
                                                         rqk, sv, dve, dpre);
  else
    k_qkv_post_bwd<T><<<cdiv(warps, WPB), 256, 0, s>>>(dqkv, qkv, ldq, ve_table, tok0, pos, sin_t, cos_t, N, H, Hkv,
                                                      hd, rqk, sv, dve, dpre);
  KERNEL_CHECK();
  return 0;
}
template <typename T>
int Stream<T>::ve_gate_bwd(const T* xn1, int D, const float* dpre, const float* ve_gate, T* dxn, int N, int Hkv,
                           float* partial, int* nblocks_out, cudaStream_t s) {
  int nb = cdiv(N, 256);
  k_ve_gate_bwd<T><<<nb, 256, sizeof(float) * 256 * Hkv, s>>>(xn1, D, dpre, ve_gate, dxn, N, Hkv, partial);
  KERNEL_CHECK();
  *nblocks_out = nb;
  return 0;
}
template <typename T>
int Stream<T>::norm_bwd_resid(const T* dy, const T* y, const float* r, const T* resid, T* out, int N, int D,
                              cudaStream_t s) {
  DISPATCH_V(D % VecN<T>::n == 0, k_norm_bwd_resid<T, V><<<row_grid(N), 256, 0, s>>>(dy, y, r, resid, out, N, D);)
  KERNEL_CHECK();
  return 0;
}
template <typename T>
int Stream<T>::mix_bwd(const T* dx_in, T* dx, const T* dxn, const T* xn1, const float* r1, const T* xin, const T* x0,
                       const float* lam_b, const float* lam_x0, T* dx0, bool first, int N, int D, float* partial,
                       int* nblocks_out, cudaStream_t s) {
  int nb = red_grid(N);
  DISPATCH_V(D % VecN<T>::n == 0, k_mix_bwd<T, V><<<nb, 256, 0, s>>>(dx_in, dx, dxn, xn1, r1, xin, x0, lam_b, lam_x0, dx0,
                                                                    first ? 1 : 0, N, D, partial);)
  KERNEL_CHECK();
  *nblocks_out = nb;
  return 0;
}
template <typename T>
int Stream<T>::backout_norm(const T* xl, const T* xb, const float* lam_y, T*, T* xnf, float* rf, int N, int D,
                            float eps, cudaStream_t s) {
  DISPATCH_V(D % VecN<T>::n == 0, k_backout_norm<T, V><<<row_grid(N), 256, 0, s>>>(xl, xb, lam_y, xnf, rf, N, D, eps);)
  KERNEL_CHECK();
  return 0;
}
template <typename T>
int Stream<T>::head_bwd(const T* dxnf, const T* xnf, const float* rf, const T* xb, T* dxf, int N, int D,
                        float* partial, int* nblocks_out, cudaStream_t s) {
  int nb = red_grid(N);
  DISPATCH_V(D % VecN<T>::n == 0, k_head_bwd<T, V><<<nb, 256, 0, s>>>(dxnf, xnf, rf, xb, dxf, N, D, partial);)
  KERNEL_CHECK();
  *nblocks_out = nb;
  return 0;
}
template <typename T> int Stream<T>::axpy(T* y, const T* x, const float* a_dev, float a_mul, long long n, cudaStream_t s) {
  constexpr int V = VecN<T>::n;
  if (n % V == 0 && aligned16(y) && aligned16(x)) {
    const int nb = (int)std::min<long long>(cdiv(n / V, 256), 148 * 8);
    k_axpy_vec<T, V><<<nb, 256, 0, s>>>(y, x, a_dev, a_mul, n / V);
  } else {
    const int nb = (int)std::min<long long>(cdiv(n, 256), 148 * 16);
    k_axpy<T><<<nb, 256, 0, s>>>(y, x, a_dev, a_mul, n);
  }
  KERNEL_CHECK();
  return 0;
}
template <typename T> int Stream<T>::add(T* y, const T* x, long long n, cudaStream_t s) {
  return axpy(y, x, nullptr, 1.f, n, s);
}
template <typename T>
int Stream<T>::smear_gate_bwd(const T* dx0, const T* xe, const float* sg, const float* lam_s, int N, int Tlen, int D,
                              float* dpre, float* partial, int* nblocks_out, cudaStream_t s) {
  int nb = red_grid(N);
  DISPATCH_V(D % VecN<T>::n == 0, k_smear_gate_bwd<T, V><<<nb, 256, 0, s>>>(dx0, xe, sg, lam_s, N, Tlen, D, dpre, partial);)
  KERNEL_CHECK();
  *nblocks_out = nb;
  return 0;
}
template <typename T>
int Stream<T>::embed_bwd(const T* dx0, const T* table, const int* tok0, const T* xe, const float* sg,
                         const float* dpre, const float* w_s, const float* lam_s, int N, int Tlen, int D, float eps,
                         T* dE, cudaStream_t s) {
  DISPATCH_V(D % VecN<T>::n == 0, k_embed_bwd<T, V><<<row_grid(N), 256, 0, s>>>(dx0, table, tok0, xe, sg, dpre, w_s,
                                                                               lam_s, N, Tlen, D, eps, dE);)
  KERNEL_CHECK();
  return 0;
}
template <typename T>
int Stream<T>::xent_rows(const float* logits, long long ldl, const int* tgt0, int n, int V, float w,
                         const float* w_dev, T* dlogit, long long lddl, float* loss_rows, cudaStream_t s) {
  k_xent_rows<T><<<n, 256, 0, s>>>(logits, ldl, tgt0, V, w, w_dev, dlogit, lddl, loss_rows);
  KERNEL_CHECK();
  return 0;
}
template <typename T> int Stream<T>::cast_from_f32(const float* src, T* dst, long long n, cudaStream_t s) {
  int nb = (int)std::min<long long>(cdiv(n, 256), 148 * 32);
  k_cast<T><<<nb, 256, 0, s>>>(src, dst, n);
  KERNEL_CHECK();
  return 0;
}
template <typename T>
int Stream<T>::pack_qkv(const float* wq, const float* wk, const float* wv, T* dst, int D, int kv, cudaStream_t s) {
  long long n = (long long)D * (D + 2 * kv);
  int nb = (int)std::min<long long>(cdiv(n, 256), 148 * 32);
  k_pack_qkv<T><<<nb, 256, 0, s>>>(wq, wk, wv, dst, D, kv);
  KERNEL_CHECK();
  return 0;
}
template struct Stream<float>;
template struct Stream<bf16>;

int sum_rows_to_scalar(const float* rows, int n, float* out, const int* tgt0, int* n_valid_out, float scale_by_valid,
                       cudaStream_t s) {
  k_sum_rows<<<1, 1024, 0, s>>>(rows, n, out, tgt0, n_valid_out, scale_by_valid);
  KERNEL_CHECK();
  return 0;
}
int reduce_partials(const float* partial, int nrow, int ncol, float* out, const float* scale_dev, float scale,
                    bool accumulate, cudaStream_t s) {
  k_reduce_partials<<<cdiv(ncol, 8), 256, 0, s>>>(partial, nrow, ncol, out, scale_dev, scale, accumulate ? 1 : 0);
  KERNEL_CHECK();
  return 0;
}
int xent_finalize(const float2* stats, int ntile, const float* tz, const int* tgt0, int n, float* lse,
                  float* loss_rows, cudaStream_t s) {
  k_xent_finalize<<<cdiv(n, 8), 256, 0, s>>>(stats, ntile, tz, tgt0, n, lse, loss_rows);
  KERNEL_CHECK();
  return 0;
}
int xent_dlogit_inplace(void* logits_bf16, long long ld, const float* lse_rows, const int* tgt0, int n, int V, float w,
                        const float* w_dev, cudaStream_t s) {
  if ((ld & 7) || (V & 7)) return femto_fail(FEMTO_ERR_ALIGN, "xent_dlogit_inplace: row pitch and vocabulary must be multiples of 8");
  k_xent_dlogit_inplace<<<dim3(cdiv(V, 8192), n), 256, 0, s>>>(reinterpret_cast<bf16*>(logits_bf16), ld, lse_rows, tgt0, V, w, w_dev);
  KERNEL_CHECK();
  return 0;
}
namespace {
// z = 15 tanh(x / 15) in place (src/gpt.jl:12)
__global__ void __launch_bounds__(256) k_softcap(float* __restrict__ x, long long n) {
  pdl_trigger();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    x[i] = 15.f * tanhf(x[i] * (1.f / 15.f));
}
}  // namespace
int softcap_inplace(float* x, long long n, cudaStream_t s) {
  k_softcap<<<(int)std::min<long long>(cdiv(n, 256), 148 * 16), 256, 0, s>>>(x, n);
  KERNEL_CHECK();
  return 0;
}
int fill_zero(void* p, size_t bytes, cudaStream_t s) {
  cudaError_t e = cudaMemsetAsync(p, 0, bytes, s);
  if (e != cudaSuccess) return femto_fail((int)e, "cudaMemsetAsync failed: %s", cudaGetErrorString(e));
  return 0;
}
