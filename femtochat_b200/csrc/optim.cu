// MuonAdamW (src/optim.jl:318-440): AdamW as one fused pass per flat range (src/optim.jl:33-39,
// 75-87; GPU form ext/FemtoChatCUDAExt.jl:99-106) and Muon (src/optim.jl:198-248) with the Polar
// Express chain (src/optim.jl:131-149) run as batched GEMMs on the stacked matrices in their
// stored [in][out] orientation, so no transposes or gather/scatter copies of Theta are needed.
#include <math.h>

#include <algorithm>
#include <vector>

#include "model.cuh"
#include "streaming.cuh"

struct AdamGroup {
  long long off, n, moff; float alpha, b1, b2, eps, lam; int t; bool shard = false;
  void* shadow = nullptr;   // compute-type copy of this range kept by the model (tables only), same element order
};
struct MuonGroup {
  std::vector<long long> offs;
  std::vector<int> layers;      // block of each matrix (ascending)
  std::vector<void*> shadow;    // host copies of d_shadow / d_shadow_ld
  std::vector<int> shadow_ld;
  int k0 = 0, k1 = 0;           // the matrices this rank updates (all of them unless sharded)
  int out = 0, in = 0;          // Julia shape (m, n) = (out, in); stored row-major [in][out]
  long long moff = 0, voff = 0; // into muon_m / muon_v
  float alpha, mu, b2, lam;
  long long* d_offs = nullptr;
  // where the model keeps the compute-type copy of each matrix: base pointer (of the handle's compute type) and row
  // pitch in elements (Q, K and V of a block live side by side in one packed matrix)
  void** d_shadow = nullptr;
  int* d_shadow_ld = nullptr;
};

struct femto_optimizer {
  femto_handle* h = nullptr;
  femto_optimizer_config cfg;
  std::vector<AdamGroup> adam;
  std::vector<MuonGroup> muon;
  float *adam_m = nullptr, *adam_v = nullptr, *muon_m = nullptr, *muon_v = nullptr;
  char* ws = nullptr;  // X fp32 stack, two compute-type stacks, A, B2, small vectors
  float* X = nullptr; void *Xa = nullptr, *Xb = nullptr, *A = nullptr, *B2 = nullptr;
  float *vec = nullptr, *fac = nullptr, *tot = nullptr;
  // owner-sharded update (data parallel): which part of every group this rank updates, and the ranges to publish
  int shard_rank = 0, shard_world = 1;
  std::vector<long long> gathers;   // (offset, count per rank)
  std::vector<long long> bcasts;    // (offset, count, owner)
  std::vector<long long> gaps;      // (offset, count): what lies between them, replicated
  std::vector<long long> foreign;   // (offset, count): what this rank clears before the exchange of Theta
  // the same for the model's compute-type weights: (byte offset from weights_begin, bytes) of what other ranks own
  std::vector<size_t> foreign_weights;
  int exchange_mode = 0;            // 0: fp32 Theta after every update; 1: compute-type weights only (Theta on demand)
};

namespace {

template <typename S>
__global__ void __launch_bounds__(256) k_adamw(float* __restrict__ theta, const float* __restrict__ delta,
                                               float* __restrict__ m, float* __restrict__ v, long long n, float alpha,
                                               float b1, float b2, float eps, float lam, float inv_c1, float inv_c2,
                                               float inv_nt, S* __restrict__ shadow) {
  pdl_trigger();
  // four elements per thread, a block apart: the sixteen loads are issued before the arithmetic, which is what
  // keeps enough bytes in flight (group offsets are arbitrary, so no wider-than-4-byte access is assumed)
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < n; i0 += 4 * stride) {
    float g[4], mo[4], vo[4], th[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const long long i = i0 + u * stride;
      if (i < n) { g[u] = delta[i]; mo[u] = m[i]; vo[u] = v[i]; th[u] = theta[i]; }
    }
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const long long i = i0 + u * stride;
      if (i >= n) continue;
      const float gg = g[u] * inv_nt;
      const float mm = b1 * mo[u] + (1.f - b1) * gg;
      const float vv = b2 * vo[u] + (1.f - b2) * gg * gg;
      m[i] = mm;
      v[i] = vv;
      const float t = th[u] * (1.f - alpha * lam);
      // Bias corrections as multiplications and the quotient as a correctly rounded reciprocal times the numerator
      // (within 2 ulp of the divisions): an IEEE division takes a slow path, about a hundred instructions, whenever
      // its numerator is zero or tiny, which is the steady state of every embedding row whose token was not in the
      // batch (measured 0.19 ms per 42 M-element table with O(1) gradients, 0.32 ms with zero gradients).
      const float tn = t - alpha * ((mm * inv_c1) * __frcp_rn(sqrtf(vv * inv_c2) + eps));
      theta[i] = tn;
      // the model's compute-type copy of the weights is refreshed in the same pass (2 more bytes per parameter
      // instead of a separate read-and-cast pass over Theta)
      if (shadow) shadow[i] = from_f<S>(tn);
    }
  }
}

// Every small AdamW group (the per-block scalars, the smear gate, ...) in ONE launch: block b takes group b.
struct SmallAdam { long long off, moff; int n; float alpha, b1, b2, eps, lam, c1, c2; };
constexpr int SMALL_BATCH = 64;                 // groups per launch: the batch travels in the kernel's parameter space
struct SmallBatch { SmallAdam g[SMALL_BATCH]; };
__global__ void __launch_bounds__(128) k_adamw_small(float* __restrict__ theta, const float* __restrict__ delta,
                                                     float* __restrict__ m, float* __restrict__ v,
                                                     const __grid_constant__ SmallBatch batch, float inv_nt) {
  pdl_trigger();
  const SmallAdam& g = batch.g[blockIdx.x];
  for (int i = threadIdx.x; i < g.n; i += 128) {
    const float gg = delta[g.off + i] * inv_nt;
    const float mm = g.b1 * m[g.moff + i] + (1.f - g.b1) * gg;
    const float vv = g.b2 * v[g.moff + i] + (1.f - g.b2) * gg * gg;
    m[g.moff + i] = mm;
    v[g.moff + i] = vv;
    const float t = theta[g.off + i] * (1.f - g.alpha * g.lam);
    theta[g.off + i] = t - g.alpha * (mm / g.c1) / (sqrtf(vv / g.c2) + g.eps);
  }
}

// mom = mu*mom + (1-mu)*g ; X = (1-mu)*g + mu*mom  (src/optim.jl:206-207)
__global__ void __launch_bounds__(256) k_muon_momentum(const float* __restrict__ delta, const long long* __restrict__ offs,
                                                       float* __restrict__ mom, float* __restrict__ X, long long per,
                                                       float mu, float inv_nt) {
  pdl_trigger();
  const int k = blockIdx.y;
  const float* g = delta + offs[k];
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per; i += (long long)gridDim.x * blockDim.x) {
    float gv = g[i] * inv_nt;
    float mm = mu * mom[k * per + i] + (1.f - mu) * gv;
    mom[k * per + i] = mm;
    X[k * per + i] = (1.f - mu) * gv + mu * mm;
  }
}

// vec[k][o] = sum_i X[k][i][o]^2 (thread per column, rows in order)
template <typename T>
__global__ void __launch_bounds__(256) k_sumsq_cols(const T* __restrict__ X, int in, int out, float* __restrict__ vec) {
  pdl_trigger();
  const int k = blockIdx.y;
  const int o = blockIdx.x * 256 + threadIdx.x;
  if (o >= out) return;
  const T* p = X + (long long)k * in * out + o;
  // eight independent partial sums (rows i mod 8), combined in a fixed order: eight loads in flight per thread
  float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  int i = 0;
  for (; i + 8 <= in; i += 8) {
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; u++) v[u] = to_f<T>(p[(long long)(i + u) * out]);
#pragma unroll
    for (int u = 0; u < 8; u++) a[u] += v[u] * v[u];
  }
  for (; i < in; i++) { float v = to_f<T>(p[(long long)i * out]); a[i & 7] += v * v; }
  vec[(long long)k * out + o] = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
}
// vec[k][i] = sum_o X[k][i][o]^2 (warp per row)
template <typename T>
__global__ void __launch_bounds__(256) k_sumsq_rows(const T* __restrict__ X, int in, int out, float* __restrict__ vec) {
  pdl_trigger();
  const int k = blockIdx.y;
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (i >= in) return;
  const T* p = X + ((long long)k * in + i) * out;
  float acc = 0.f;
  for (int o = lane; o < out; o += 32) { float v = to_f<T>(p[o]); acc += v * v; }
  acc = warp_sum(acc);
  if (lane == 0) vec[(long long)k * in + i] = acc;
}

// MuonEq + Polar-Express normalisation factors (src/optim.jl:210-212,135-136), one block per matrix:
// fac[k][o] = sqrt(old/m)/max(sqrt(row[o]),1e-6) / (1.01*sqrt(sum_o fac0^2*row[o]) + 1e-6)
__global__ void __launch_bounds__(256) k_muoneq_factors(const float* __restrict__ vec, int out, float* __restrict__ fac) {
  pdl_trigger();
  __shared__ float red[256];
  const int k = blockIdx.x;
  const float* row = vec + (long long)k * out;
  float acc = 0.f;
  for (int o = threadIdx.x; o < out; o += 256) acc += row[o];
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) { if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s]; __syncthreads(); }
  const float old = red[0];
  __syncthreads();
  const float num = sqrtf(old / (float)out);
  acc = 0.f;
  for (int o = threadIdx.x; o < out; o += 256) {
    float f = num / fmaxf(sqrtf(row[o]), 1e-6f);
    acc += f * f * row[o];
  }
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) { if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s]; __syncthreads(); }
  const float scale = 1.01f * sqrtf(red[0]) + 1e-6f;
  for (int o = threadIdx.x; o < out; o += 256) fac[(long long)k * out + o] = num / fmaxf(sqrtf(row[o]), 1e-6f) / scale;
}

template <typename T>
__global__ void __launch_bounds__(256) k_scale_cols_cast(const float* __restrict__ X, const float* __restrict__ fac,
                                                         T* __restrict__ Y, long long per, int out) {
  pdl_trigger();
  const int k = blockIdx.y;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per; i += (long long)gridDim.x * blockDim.x)
    Y[k * per + i] = from_f<T>(X[k * per + i] * fac[(long long)k * out + (int)(i % out)]);
}
// The same with four adjacent columns per thread (out a multiple of 4, 16-byte aligned stacks): 16-byte loads, 32-bit
// index arithmetic inside a matrix.
template <typename T>
__global__ void __launch_bounds__(256) k_scale_cols_cast4(const float* __restrict__ X, const float* __restrict__ fac,
                                                          T* __restrict__ Y, int per4, int out4) {
  pdl_trigger();
  const int k = blockIdx.y;
  const float4* x4 = reinterpret_cast<const float4*>(X) + (long long)k * per4;
  const float4* f4 = reinterpret_cast<const float4*>(fac) + (long long)k * out4;
  T* y = Y + (long long)k * per4 * 4;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < per4; i += gridDim.x * blockDim.x) {
    const float4 v = x4[i], f = f4[i % out4];
    const float r[4] = {v.x * f.x, v.y * f.y, v.z * f.z, v.w * f.w};
    if constexpr (sizeof(T) == 2) {
      uint2 q;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
      h[0] = __floats2bfloat162_rn(r[0], r[1]); h[1] = __floats2bfloat162_rn(r[2], r[3]);
      *reinterpret_cast<uint2*>(y + 4ll * i) = q;
    } else {
      *reinterpret_cast<float4*>(y + 4ll * i) = make_float4(r[0], r[1], r[2], r[3]);
    }
  }
}

// Muon+ and NorMuon factors (src/optim.jl:218-233), one block per matrix.  vec = sums of X^2 along
// the reduced axis (length dim, each over dsize elements); v is the persistent second moment.
__global__ void __launch_bounds__(256) k_normuon_factors(const float* __restrict__ vec, int dim, int dsize, int rmin,
                                                         float b2, float* __restrict__ v, float* __restrict__ fac) {
  pdl_trigger();
  __shared__ float red[256];
  const int k = blockIdx.x;
  const float* S = vec + (long long)k * dim;
  float* vv = v + (long long)k * dim;
  float acc = 0.f;
  for (int j = threadIdx.x; j < dim; j += 256) acc += S[j];
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) { if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s]; __syncthreads(); }
  const float old0 = red[0];
  __syncthreads();
  const float f1 = sqrtf((float)rmin) / fmaxf(sqrtf(old0), 1e-6f);
  const float old = f1 * f1 * old0;
  acc = 0.f;
  for (int j = threadIdx.x; j < dim; j += 256) {
    float vm = f1 * f1 * S[j] / (float)dsize;
    float nv = b2 * vv[j] + (1.f - b2) * vm;
    vv[j] = nv;
    float st = rsqrtf(fmaxf(nv, 1e-10f));
    acc += (float)dsize * vm * st * st;
  }
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) { if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s]; __syncthreads(); }
  const float g = f1 * sqrtf(old) / fmaxf(sqrtf(red[0]), 1e-10f);
  for (int j = threadIdx.x; j < dim; j += 256) fac[(long long)k * dim + j] = g * rsqrtf(fmaxf(vv[j], 1e-10f));
}

// theta -= eta*X + eta*lam*theta*[X*theta >= 0]  (src/optim.jl:244-245; ext/FemtoChatCUDAExt.jl:108-119)
template <typename T, typename S>
__global__ void __launch_bounds__(256) k_muon_update(float* __restrict__ theta, const long long* __restrict__ offs,
                                                     const T* __restrict__ X, const float* __restrict__ fac,
                                                     long long per, int out, int by_col, int dim, float eta, float lam,
                                                     void* const* __restrict__ shadow, const int* __restrict__ shadow_ld) {
  pdl_trigger();
  const int k = blockIdx.y;
  float* th = theta + offs[k];
  S* sh = shadow ? reinterpret_cast<S*>(shadow[k]) : nullptr;
  const int sld = shadow ? shadow_ld[k] : 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per; i += (long long)gridDim.x * blockDim.x) {
    const int col = (int)(i % out), row = (int)(i / out);
    int j = by_col ? col : row;
    float x = to_f<T>(X[k * per + i]) * fac[(long long)k * dim + j];
    float t = th[i];
    const float tn = t - (eta * x + eta * lam * t * ((x * t) >= 0.f ? 1.f : 0.f));
    th[i] = tn;
    if (sh) sh[(long long)row * sld + col] = from_f<S>(tn);   // the model's compute-type copy, refreshed in the same pass
  }
}

// The same with two adjacent columns per thread (matrices of even width; every range of Theta starts at an even
// element offset, so the pairs are 8-byte aligned), 32-bit index arithmetic inside a matrix.  by_col: the factor
// belongs to the column.
template <typename T, typename S>
__global__ void __launch_bounds__(256) k_muon_update2(float* __restrict__ theta, const long long* __restrict__ offs,
                                                      const T* __restrict__ X, const float* __restrict__ fac,
                                                      int per2, int out2, int by_col, int dim, float eta, float lam,
                                                      void* const* __restrict__ shadow, const int* __restrict__ shadow_ld) {
  pdl_trigger();
  const int k = blockIdx.y;
  float2* th = reinterpret_cast<float2*>(theta + offs[k]);
  S* sh = shadow ? reinterpret_cast<S*>(shadow[k]) : nullptr;
  const int sld = shadow ? shadow_ld[k] : 0;
  const T* x = X + (long long)k * per2 * 2;
  const float* fk = fac + (long long)k * dim;
  const int stride = gridDim.x * blockDim.x;
  for (int i0 = blockIdx.x * blockDim.x + threadIdx.x; i0 < per2; i0 += 4 * stride) {
    float2 t2[4], xv[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const int i = i0 + u * stride;
      if (i >= per2) continue;
      t2[u] = th[i];
      if constexpr (sizeof(T) == 2) {
        const __nv_bfloat162 q = *reinterpret_cast<const __nv_bfloat162*>(x + 2ll * i);
        xv[u] = make_float2(__bfloat162float(q.x), __bfloat162float(q.y));
      } else {
        xv[u] = *reinterpret_cast<const float2*>(x + 2ll * i);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const int i = i0 + u * stride;
      if (i >= per2) continue;
      const int row = i / out2, c2 = i % out2;
      float2 f;
      if (by_col) f = *reinterpret_cast<const float2*>(fk + 2 * c2);
      else { const float q = fk[row]; f = make_float2(q, q); }
      const float x0 = xv[u].x * f.x, x1 = xv[u].y * f.y;
      const float r0 = t2[u].x - (eta * x0 + eta * lam * t2[u].x * ((x0 * t2[u].x) >= 0.f ? 1.f : 0.f));
      const float r1 = t2[u].y - (eta * x1 + eta * lam * t2[u].y * ((x1 * t2[u].y) >= 0.f ? 1.f : 0.f));
      th[i] = make_float2(r0, r1);
      if (sh) {
        S* dst = sh + (long long)row * sld + 2 * c2;
        if constexpr (sizeof(S) == 2) *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(r0, r1);
        else *reinterpret_cast<float2*>(dst) = make_float2(r0, r1);
      }
    }
  }
}

inline int egrid(long long n) { return (int)std::min<long long>(cdiv(n, 256), 148 * 8); }

}  // namespace

// shadow (may be null): compute-type copy of the range, of type bf16 when shadow_bf16 else float
static int adamw_launch_shadow(float* theta, const float* delta, float* m, float* v, long long n, float alpha, float b1,
                               float b2, float eps, float lam, int t, float n_tokens, void* shadow, bool shadow_bf16,
                               cudaStream_t s) {
  const float c1 = 1.f - powf(b1, (float)t), c2 = 1.f - powf(b2, (float)t);
  if (shadow_bf16) k_adamw<bf16><<<egrid(n), 256, 0, s>>>(theta, delta, m, v, n, alpha, b1, b2, eps, lam, 1.f / c1, 1.f / c2, 1.f / n_tokens, (bf16*)shadow);
  else k_adamw<float><<<egrid(n), 256, 0, s>>>(theta, delta, m, v, n, alpha, b1, b2, eps, lam, 1.f / c1, 1.f / c2, 1.f / n_tokens, (float*)shadow);
  KERNEL_CHECK();
  return 0;
}
int adamw_launch(float* theta, const float* delta, float* m, float* v, long long n, float alpha, float b1, float b2,
                 float eps, float lam, int t, float n_tokens, cudaStream_t s) {
  return adamw_launch_shadow(theta, delta, m, v, n, alpha, b1, b2, eps, lam, t, n_tokens, nullptr, false, s);
}

// C[b][i][j] = C[b][j][i] for i > j on a stack of r x r matrices: completes a symmetric product of which only the
// tiles touching the upper triangle were computed.  64 x 64 tiles through shared memory, one block per tile pair.
template <typename T>
__global__ void __launch_bounds__(256) k_mirror_upper(T* __restrict__ C, int r, long long stride, int nb) {
  pdl_trigger();
  __shared__ float tile[64][65];
  // blockIdx.x enumerates the tile pairs (bi >= bj) of the lower triangle, 64 x 64 elements each
  int bi = (int)((sqrtf(8.f * blockIdx.x + 1.f) - 1.f) * 0.5f);
  while ((bi + 1) * (bi + 2) / 2 <= (int)blockIdx.x) bi++;
  while (bi * (bi + 1) / 2 > (int)blockIdx.x) bi--;
  const int bj = blockIdx.x - bi * (bi + 1) / 2;
  if (bi >= nb) return;
  T* M = C + (long long)blockIdx.y * stride;
  if ((r & 1) == 0) {
    // two adjacent columns per thread: a warp moves one 64-element row (128 bytes of bf16) per access
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (int y = w; y < 64; y += 8) {            // source tile: rows bj*64.., cols bi*64..
      const int sr = bj * 64 + y, sc = bi * 64 + 2 * lane;
      float a = 0.f, b = 0.f;
      if (sr < r && sc < r) {                    // r even: sc + 1 < r as well
        const T* src = M + (long long)sr * r + sc;
        if constexpr (sizeof(T) == 2) {
          const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(src);
          a = __bfloat162float(v.x); b = __bfloat162float(v.y);
        } else {
          const float2 v = *reinterpret_cast<const float2*>(src);
          a = v.x; b = v.y;
        }
      }
      tile[y][2 * lane] = a; tile[y][2 * lane + 1] = b;
    }
    __syncthreads();
    for (int y = w; y < 64; y += 8) {
      const int dr = bi * 64 + y, dc = bj * 64 + 2 * lane;
      if (dr >= r || dc >= r || dr <= dc) continue;      // on or above the diagonal: keep what the GEMM wrote
      T* dst = M + (long long)dr * r + dc;
      const float a = tile[2 * lane][y], b = tile[2 * lane + 1][y];
      if (dr > dc + 1) {
        if constexpr (sizeof(T) == 2) *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(a, b);
        else *reinterpret_cast<float2*>(dst) = make_float2(a, b);
      } else {
        dst[0] = from_f<T>(a);                            // dr == dc + 1: the second column is the diagonal
      }
    }
    return;
  }
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  for (int y = ty; y < 64; y += 4) {            // source tile: rows bj*64.., cols bi*64..
    const int sr = bj * 64 + y, sc = bi * 64 + tx;
    tile[y][tx] = (sr < r && sc < r) ? to_f<T>(M[(long long)sr * r + sc]) : 0.f;
  }
  __syncthreads();
  for (int y = ty; y < 64; y += 4) {
    const int dr = bi * 64 + y, dc = bj * 64 + tx;
    if (dr < r && dc < r && dr > dc) M[(long long)dr * r + dc] = from_f<T>(tile[tx][y]);
  }
}
template <typename T> int mirror_upper(T* C, int r, long long stride, int k, cudaStream_t s) {
  const int nb = cdiv(r, 64);
  k_mirror_upper<T><<<dim3(nb * (nb + 1) / 2, k), 256, 0, s>>>(C, r, stride, nb);
  KERNEL_CHECK();
  return 0;
}

// Polar Express on a stack S[k][in][out] of type T, in place (result left in S).  scratch: S2 like S,
// A and B2 [k][r][r].
template <typename T>
int newton_schulz_t(T* S, T* S2, T* A, T* B2, int k, int in, int out, const float* coeffs, int steps, void* ws,
                    size_t ws_bytes, unsigned int* status, cudaStream_t s) {
  const bool tall = out > in;  // Julia m > n: iterate on S as stored (rows = in)
  const int r = std::min(in, out);
  const long long per = (long long)in * out, rr = (long long)r * r;
  T* cur = S;
  T* nxt = S2;
  for (int t = 0; t < steps; t++) {
    const float a = coeffs[3 * t], b = coeffs[3 * t + 1], c = coeffs[3 * t + 2];
    GemmArgs g;
    g.ws = ws; g.ws_bytes = ws_bytes; g.status = status; g.batch = k;
    // A = X X^T
    g.A = cur; g.B = cur; g.lda = out; g.ldb = out; g.strideA = per; g.strideB = per;
    g.a_kmajor = tall; g.b_kmajor = tall;
    g.C = A; g.ldc = r; g.strideC = rr; g.M = r; g.N = r; g.K = tall ? out : in; g.epi = EPI_STORE;
    g.upper_only = true;   // X X^T is symmetric: compute the tiles on and above the diagonal, mirror the rest
    FEMTO_TRY(gemm<T>(g, s));
    FEMTO_TRY(mirror_upper<T>(A, r, rr, k, s));
    // B2 = b A + c A A
    GemmArgs g2;
    g2.ws = ws; g2.ws_bytes = ws_bytes; g2.status = status; g2.batch = k;
    g2.A = A; g2.B = A; g2.lda = r; g2.ldb = r; g2.strideA = rr; g2.strideB = rr; g2.a_kmajor = true; g2.b_kmajor = true;
    g2.C = B2; g2.ldc = r; g2.strideC = rr; g2.M = r; g2.N = r; g2.K = r;
    g2.epi = EPI_AXPBY; g2.aux = A; g2.ldaux = r; g2.strideAux = rr; g2.alpha = b; g2.beta = c;
    g2.upper_only = true;  // a polynomial of a symmetric matrix is symmetric
    FEMTO_TRY(gemm<T>(g2, s));
    FEMTO_TRY(mirror_upper<T>(B2, r, rr, k, s));
    // X' = a X + B2 X   (stored orientation: S' = a S + B2 S when tall, S' = a S + S B2 otherwise)
    GemmArgs g3;
    g3.ws = ws; g3.ws_bytes = ws_bytes; g3.status = status; g3.batch = k;
    if (tall) {
      g3.A = B2; g3.lda = r; g3.strideA = rr; g3.a_kmajor = true;
      g3.B = cur; g3.ldb = out; g3.strideB = per; g3.b_kmajor = false;
      g3.M = r; g3.N = out; g3.K = r;
    } else {
      g3.A = cur; g3.lda = out; g3.strideA = per; g3.a_kmajor = true;
      g3.B = B2; g3.ldb = r; g3.strideB = rr; g3.b_kmajor = true;
      g3.M = in; g3.N = out; g3.K = r;
    }
    g3.C = nxt; g3.ldc = out; g3.strideC = per;
    g3.epi = EPI_AXPBY; g3.aux = cur; g3.ldaux = out; g3.strideAux = per; g3.alpha = a; g3.beta = 1.f;
    FEMTO_TRY(gemm<T>(g3, s));
    std::swap(cur, nxt);
  }
  if (cur != S) CUDA_TRY(cudaMemcpyAsync(S, cur, sizeof(T) * per * k, cudaMemcpyDeviceToDevice, s));
  return 0;
}
template int newton_schulz_t<float>(float*, float*, float*, float*, int, int, int, const float*, int, void*, size_t,
                                    unsigned int*, cudaStream_t);
template int newton_schulz_t<bf16>(bf16*, bf16*, bf16*, bf16*, int, int, int, const float*, int, void*, size_t,
                                   unsigned int*, cudaStream_t);

template <typename T> static int muon_group_step(femto_optimizer* o, MuonGroup& g, float* theta, const float* delta,
                                                  float alpha, float mu, float lam, float nt, cudaStream_t s) {
  femto_handle* h = o->h;
  const int k = g.k1 - g.k0, in = g.in, out = g.out;
  if (k <= 0) return 0;
  const long long per = (long long)in * out;
  const long long* d_offs = g.d_offs + g.k0;
  float* mom = o->muon_m + g.moff + (long long)g.k0 * per;
  float* v = o->muon_v + g.voff + (long long)g.k0 * (out >= in ? out : in);
  dim3 eg(egrid(per), k);
  k_muon_momentum<<<eg, 256, 0, s>>>(delta, d_offs, mom, o->X, per, mu, 1.f / nt);
  KERNEL_CHECK();
  k_sumsq_cols<float><<<dim3(cdiv(out, 256), k), 256, 0, s>>>(o->X, in, out, o->vec);
  KERNEL_CHECK();
  k_muoneq_factors<<<k, 256, 0, s>>>(o->vec, out, o->fac);
  KERNEL_CHECK();
  if ((out & 3) == 0 && per / 4 < (1ll << 30)) {
    k_scale_cols_cast4<T><<<dim3((unsigned)std::min<long long>(cdiv(per / 4, 256), 148 * 8), k), 256, 0, s>>>(o->X, o->fac, (T*)o->Xa, (int)(per / 4), out / 4);
  } else {
    k_scale_cols_cast<T><<<eg, 256, 0, s>>>(o->X, o->fac, (T*)o->Xa, per, out);
  }
  KERNEL_CHECK();
  FEMTO_TRY(newton_schulz_t<T>((T*)o->Xa, (T*)o->Xb, (T*)o->A, (T*)o->B2, k, in, out, o->cfg.ns_coeffs,
                               o->cfg.ns_steps, h->gemm_ws, h->gemm_ws_bytes, h->status, s));
  // NorMuon reduces over Julia dim 2 (in) when m >= n, else over dim 1 (out)
  const bool by_col = out >= in;
  const int dim = by_col ? out : in, dsize = by_col ? in : out;
  if (by_col) k_sumsq_cols<T><<<dim3(cdiv(out, 256), k), 256, 0, s>>>((const T*)o->Xa, in, out, o->vec);
  else k_sumsq_rows<T><<<dim3(cdiv(in, 8), k), 256, 0, s>>>((const T*)o->Xa, in, out, o->vec);
  KERNEL_CHECK();
  k_normuon_factors<<<k, 256, 0, s>>>(o->vec, dim, dsize, std::min(in, out), g.b2, v, o->fac);
  KERNEL_CHECK();
  const float eta = alpha * sqrtf(std::max(1.f, (float)out / (float)in));
  void* const* sh = g.d_shadow ? g.d_shadow + g.k0 : nullptr;
  const int* shld = g.d_shadow_ld ? g.d_shadow_ld + g.k0 : nullptr;
  bool pairs = (out & 1) == 0 && per / 2 < (1ll << 30) && (reinterpret_cast<uintptr_t>(theta) & 7u) == 0;
  for (int i = g.k0; i < g.k1 && pairs; i++)
    pairs = (g.offs[i] & 1) == 0 && (g.shadow_ld[i] & 1) == 0 && (reinterpret_cast<uintptr_t>(g.shadow[i]) & (h->bf ? 3u : 7u)) == 0;
  if (pairs) {
    dim3 eg2((unsigned)std::min<long long>(cdiv(per / 2, 1024), 148 * 8), k);
    if (h->bf) k_muon_update2<T, bf16><<<eg2, 256, 0, s>>>(theta, d_offs, (const T*)o->Xa, o->fac, (int)(per / 2), out / 2, by_col ? 1 : 0, dim, eta, lam, sh, shld);
    else k_muon_update2<T, float><<<eg2, 256, 0, s>>>(theta, d_offs, (const T*)o->Xa, o->fac, (int)(per / 2), out / 2, by_col ? 1 : 0, dim, eta, lam, sh, shld);
  } else if (h->bf) {
    k_muon_update<T, bf16><<<eg, 256, 0, s>>>(theta, d_offs, (const T*)o->Xa, o->fac, per, out, by_col ? 1 : 0, dim, eta, lam, sh, shld);
  } else {
    k_muon_update<T, float><<<eg, 256, 0, s>>>(theta, d_offs, (const T*)o->Xa, o->fac, per, out, by_col ? 1 : 0, dim, eta, lam, sh, shld);
  }
  KERNEL_CHECK();
  return 0;
}

// X_out[k][in][out] = fac * Polar-Express direction: the stand-alone form of muon_direction! (src/optim.jl:198-236)
// on a contiguous stack of k fp32 gradients G[k][in][out] (the stored orientation of a Julia (out, in) matrix).
namespace {
template <typename T>
__global__ void __launch_bounds__(256) k_direction_out(const T* __restrict__ X, const float* __restrict__ fac,
                                                       float* __restrict__ out_, long long per, int out, int by_col, int dim) {
  pdl_trigger();
  const int k = blockIdx.y;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per; i += (long long)gridDim.x * blockDim.x) {
    const int j = by_col ? (int)(i % out) : (int)(i / out);
    out_[k * per + i] = to_f<T>(X[k * per + i]) * fac[(long long)k * dim + j];
  }
}
__global__ void k_stack_offsets(long long* offs, int k, long long per) {
  pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < k) offs[i] = (long long)i * per;
}
}  // namespace

template <typename T>
static int muon_direction_t(float* X_out, const float* G, float* mom, float* v, int k, int in, int out, float mu, float b2,
                            float nt, const float* coeffs, int steps, unsigned int* status, char* buf, cudaStream_t s) {
  const long long per = (long long)in * out;
  const size_t r = std::min(in, out);
  auto al = [](size_t b) { return (b + 255) & ~(size_t)255; };
  char* p = buf;
  float* X = (float*)p; p += al(4 * per * k);
  T* Xa = (T*)p; p += al(sizeof(T) * per * k);
  T* Xb = (T*)p; p += al(sizeof(T) * per * k);
  T* A = (T*)p; p += al(sizeof(T) * r * r * k);
  T* B2 = (T*)p; p += al(sizeof(T) * r * r * k);
  float* vec = (float*)p; p += al(4 * (size_t)k * std::max(in, out));
  float* fac = (float*)p; p += al(4 * (size_t)k * std::max(in, out));
  long long* offs = (long long*)p; p += al(8 * (size_t)k);
  void* ws = p;
  const size_t wsb = (size_t)160 << 20;
  k_stack_offsets<<<cdiv(k, 256), 256, 0, s>>>(offs, k, per);
  KERNEL_CHECK();
  dim3 eg(egrid(per), k);
  k_muon_momentum<<<eg, 256, 0, s>>>(G, offs, mom, X, per, mu, 1.f / nt);
  KERNEL_CHECK();
  k_sumsq_cols<float><<<dim3(cdiv(out, 256), k), 256, 0, s>>>(X, in, out, vec);
  KERNEL_CHECK();
  k_muoneq_factors<<<k, 256, 0, s>>>(vec, out, fac);
  KERNEL_CHECK();
  k_scale_cols_cast<T><<<eg, 256, 0, s>>>(X, fac, Xa, per, out);
  KERNEL_CHECK();
  FEMTO_TRY(newton_schulz_t<T>(Xa, Xb, A, B2, k, in, out, coeffs, steps, ws, wsb, status, s));
  const bool by_col = out >= in;
  const int dim = by_col ? out : in, dsize = by_col ? in : out;
  if (by_col) k_sumsq_cols<T><<<dim3(cdiv(out, 256), k), 256, 0, s>>>(Xa, in, out, vec);
  else k_sumsq_rows<T><<<dim3(cdiv(in, 8), k), 256, 0, s>>>(Xa, in, out, vec);
  KERNEL_CHECK();
  k_normuon_factors<<<k, 256, 0, s>>>(vec, dim, dsize, std::min(in, out), b2, v, fac);
  KERNEL_CHECK();
  k_direction_out<T><<<eg, 256, 0, s>>>(Xa, fac, X_out, per, out, by_col ? 1 : 0, dim);
  KERNEL_CHECK();
  return 0;
}

int muon_direction_standalone(int dtype, float* X_out, const float* G, float* mom, float* v, int k, int in, int out,
                              float mu, float b2, float n_tokens, const float* coeffs, int steps, unsigned int* status,
                              cudaStream_t s) {
  const size_t es = dtype == FEMTO_BF16 ? 2 : 4;
  const size_t per = (size_t)in * out, r = std::min(in, out);
  auto al = [](size_t b) { return (b + 255) & ~(size_t)255; };
  const size_t total = al(4 * per * k) + 2 * al(es * per * k) + 2 * al(es * r * r * k) + 2 * al(4 * (size_t)k * std::max(in, out)) +
                       al(8 * (size_t)k) + ((size_t)160 << 20) + 1024;
  char* buf = nullptr;
  FEMTO_TRY(standalone_scratch(total, &buf));
  return dtype == FEMTO_BF16 ? muon_direction_t<bf16>(X_out, G, mom, v, k, in, out, mu, b2, n_tokens, coeffs, steps, status, buf, s)
                             : muon_direction_t<float>(X_out, G, mom, v, k, in, out, mu, b2, n_tokens, coeffs, steps, status, buf, s);
}

int optimizer_state_sizes(femto_handle* h, long long* out4) {
  long long adam = 0, mm = 0, mv = 0;
  adam += (long long)h->Vp * h->d * 2;
  for (int i = 0; i < h->L; i++) {
    if (h->lp[i].ve) adam += (long long)h->Vp * h->kv;
    adam += 2;
  }
  adam += 24 + 1 + 1;
  const long long d = h->d, kv = h->kv;
  for (int i = 0; i < h->L; i++) {
    mm += d * d * 2 + kv * d * 2 + 8 * d * d;
    mv += std::max(d, d) * 2 + std::max(kv, d) * 2 + 4 * d + 4 * d;  // wq,wo: d; wk,wv: n=d (kv<=d); fc: m=4d; proj: n=4d
    if (h->lp[i].ve) { mm += h->Hkv * 12; mv += std::max(h->Hkv, 12); }
  }
  out4[0] = adam; out4[1] = adam; out4[2] = mm; out4[3] = mv;
  return 0;
}

int optimizer_create(femto_handle* h, const femto_optimizer_config* cfg, float* adam_m, float* adam_v, float* muon_m,
                     float* muon_v, femto_optimizer** out) {
  if (!h || !cfg || !adam_m || !adam_v || !muon_m || !muon_v || !out) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  if (cfg->ns_steps < 0 || cfg->ns_steps > 5) return femto_fail(FEMTO_ERR_ARG, "ns_steps must be 0..5");
  femto_optimizer* o = new femto_optimizer();
  o->h = h; o->cfg = *cfg; o->adam_m = adam_m; o->adam_v = adam_v; o->muon_m = muon_m; o->muon_v = muon_v;
  const float scale = sqrtf(768.f / (float)h->d);
  long long moff = 0;
  auto add = [&](long long off, long long n, float alpha, float b1, float b2, float lam, void* shadow = nullptr) {
    AdamGroup g{off, n, moff, alpha, b1, b2, 1e-10f, lam, 0};
    g.shadow = shadow;
    moff += n;
    o->adam.push_back(g);
  };
  // group order of src/optim.jl:333-403
  add(h->off_lm, (long long)h->Vp * h->d, cfg->unembedding_lr * scale, 0.8f, 0.96f, 0.01f, h->sh_lm);
  add(h->off_wte, (long long)h->Vp * h->d, cfg->embedding_lr * scale, 0.8f, 0.995f, 0.001f, h->sh_wte);
  for (int i = 0; i < h->L; i++) {
    const LayerP& p = h->lp[i];
    if (p.ve) add(p.ve_table, (long long)h->Vp * h->kv, 0.5f * cfg->embedding_lr * scale, 0.8f, 0.995f, 0.01f, h->lb[i].sh_ve);
    add(p.lam_b, 1, 0.01f * cfg->scalar_lr, 0.8f, 0.95f, 0.05f);
    add(p.lam_x0, 1, cfg->scalar_lr, 0.96f, 0.95f, 0.f);
  }
  add(h->off_smear, 24, cfg->smear_lr, 0.8f, 0.95f, 0.f);
  add(h->off_lam_s, 1, cfg->smear_lr, 0.8f, 0.95f, 0.f);
  add(h->off_lam_y, 1, cfg->smear_lr, 0.8f, 0.95f, 0.f);
  // Muon groups by shape, in order of first appearance (src/optim.jl:405-425)
  struct Spec { long long off; int out, in, layer; void* shadow; int shadow_ld; };
  std::vector<Spec> specs;
  const size_t es_model = h->bf ? 2 : 4;
  for (int i = 0; i < h->L; i++) {
    const LayerP& p = h->lp[i];
    const LayerBuf& l = h->lb[i];
    char* qkv = reinterpret_cast<char*>(l.sh_wqkv);   // [d][d + 2 kv]: Q | K | V side by side
    specs.push_back({p.wq, h->d, h->d, i, qkv, h->dq});
    specs.push_back({p.wk, h->kv, h->d, i, qkv + es_model * h->d, h->dq});
    specs.push_back({p.wv, h->kv, h->d, i, qkv + es_model * (h->d + h->kv), h->dq});
    specs.push_back({p.wo, h->d, h->d, i, l.sh_wo, h->d}); specs.push_back({p.fc, 4 * h->d, h->d, i, l.sh_fc, 4 * h->d});
    specs.push_back({p.proj, h->d, 4 * h->d, i, l.sh_proj, h->d});
    if (p.ve) specs.push_back({p.ve_gate, h->Hkv, 12, i, nullptr, 0});   // the gate is read from Theta in fp32
  }
  long long mo = 0, vo = 0;
  size_t max_stack = 0, max_rr = 0, max_vec = 0;
  for (const auto& sp : specs) {
    MuonGroup* g = nullptr;
    for (auto& e : o->muon) if (e.out == sp.out && e.in == sp.in) g = &e;
    if (!g) {
      MuonGroup ng; ng.out = sp.out; ng.in = sp.in; ng.alpha = cfg->matrix_lr; ng.mu = 0.95f; ng.b2 = 0.9f; ng.lam = cfg->weight_decay;
      o->muon.push_back(ng);
      g = &o->muon.back();
    }
    g->offs.push_back(sp.off);
    g->layers.push_back(sp.layer);
    g->shadow.push_back(sp.shadow);
    g->shadow_ld.push_back(sp.shadow_ld);
  }
  for (auto& g : o->muon) {
    const size_t k = g.offs.size();
    g.k0 = 0; g.k1 = (int)k;
    g.moff = mo; g.voff = vo;
    mo += (long long)k * g.in * g.out;
    vo += (long long)k * (g.out >= g.in ? g.out : g.in);
    max_stack = std::max(max_stack, k * (size_t)g.in * g.out);
    const size_t r = std::min(g.in, g.out);
    max_rr = std::max(max_rr, k * r * r);
    max_vec = std::max(max_vec, k * (size_t)std::max(g.in, g.out));
    CUDA_TRY(cudaMalloc(&g.d_offs, sizeof(long long) * k));
    CUDA_TRY(cudaMemcpy(g.d_offs, g.offs.data(), sizeof(long long) * k, cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMalloc(&g.d_shadow, sizeof(void*) * k));
    CUDA_TRY(cudaMemcpy(g.d_shadow, g.shadow.data(), sizeof(void*) * k, cudaMemcpyHostToDevice));
    CUDA_TRY(cudaMalloc(&g.d_shadow_ld, sizeof(int) * k));
    CUDA_TRY(cudaMemcpy(g.d_shadow_ld, g.shadow_ld.data(), sizeof(int) * k, cudaMemcpyHostToDevice));
  }
  const size_t es = cfg->compute_dtype == FEMTO_BF16 ? 2 : 4;
  auto al = [](size_t b) { return (b + 255) & ~(size_t)255; };
  size_t total = al(4 * max_stack) + 2 * al(es * max_stack) + 2 * al(es * max_rr) + 2 * al(4 * max_vec) + 256;
  CUDA_TRY(cudaMalloc(&o->ws, total));
  char* p = o->ws;
  o->X = (float*)p; p += al(4 * max_stack);
  o->Xa = p; p += al(es * max_stack);
  o->Xb = p; p += al(es * max_stack);
  o->A = p; p += al(es * max_rr);
  o->B2 = p; p += al(es * max_rr);
  o->vec = (float*)p; p += al(4 * max_vec);
  o->fac = (float*)p;
  *out = o;
  return 0;
}

int optimizer_destroy(femto_optimizer* o) {
  if (!o) return 0;
  for (auto& g : o->muon) { cudaFree(g.d_offs); cudaFree(g.d_shadow); cudaFree(g.d_shadow_ld); }
  cudaFree(o->ws);
  delete o;
  return 0;
}

int optimizer_step(femto_optimizer* o, float* theta, const float* delta, float eta, int has_mu, float mu,
                   int has_lambda, float lambda, float n_tokens, cudaStream_t s) {
  if (!o || !theta || !delta) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  if (!(n_tokens > 0.f)) return femto_fail(FEMTO_ERR_ARG, "n_tokens must be positive");
  const bool sharded = o->shard_world > 1;
  femto_handle* h = o->h;
  const size_t es_model = h->bf ? 2 : 4;
  // The AdamW tables are pure HBM streaming and touch nothing the Muon groups touch: on the handle's low-priority
  // stream they run under the Polar Express GEMMs of the Muon groups instead of before them.
  cudaStream_t sa = s;
  if (h->lo && !gemm_profiling()) {
    cudaEvent_t e = h->ev_fork[h->ev_next++ % femto_handle::N_FORK];
    CUDA_TRY(cudaEventRecord(e, s));
    CUDA_TRY(cudaStreamWaitEvent(h->lo, e, 0));
    sa = h->lo;
  }
  SmallBatch batch;
  int nsmall = 0;
  auto flush_small = [&]() -> int {
    if (nsmall == 0) return 0;
    k_adamw_small<<<nsmall, 128, 0, sa>>>(theta, delta, o->adam_m, o->adam_v, batch, 1.f / n_tokens);
    KERNEL_CHECK();
    nsmall = 0;
    return 0;
  };
  for (auto& g : o->adam) {  // src/optim.jl:431-433
    g.t += 1;
    if (!g.shard && !g.shadow && g.n <= 4096) {
      // the scalars and gates: all of them in one launch (the order of the groups does not matter, they are disjoint)
      SmallAdam& sg = batch.g[nsmall++];
      sg.off = g.off; sg.moff = g.moff; sg.n = (int)g.n; sg.alpha = eta * g.alpha; sg.b1 = g.b1; sg.b2 = g.b2; sg.eps = g.eps;
      sg.lam = g.lam; sg.c1 = 1.f - powf(g.b1, (float)g.t); sg.c2 = 1.f - powf(g.b2, (float)g.t);
      if (nsmall == SMALL_BATCH) FEMTO_TRY(flush_small());
      continue;
    }
    // a sharded table: this rank updates slice shard_rank of shard_world equal slices
    const long long n = g.shard ? g.n / o->shard_world : g.n, o0 = g.shard ? n * o->shard_rank : 0;
    void* shadow = g.shadow ? reinterpret_cast<char*>(g.shadow) + es_model * (size_t)o0 : nullptr;
    FEMTO_TRY(adamw_launch_shadow(theta + g.off + o0, delta + g.off + o0, o->adam_m + g.moff + o0, o->adam_v + g.moff + o0, n,
                                  eta * g.alpha, g.b1, g.b2, g.eps, g.lam, g.t, n_tokens, shadow, h->bf, sa));
  }
  FEMTO_TRY(flush_small());
  int rc = 0;
  for (auto& g : o->muon) {  // src/optim.jl:434-438
    const float m_ = has_mu ? mu : g.mu, l_ = has_lambda ? lambda : g.lam;
    if (o->cfg.compute_dtype == FEMTO_BF16) rc = muon_group_step<bf16>(o, g, theta, delta, eta * g.alpha, m_, l_, n_tokens, s);
    else rc = muon_group_step<float>(o, g, theta, delta, eta * g.alpha, m_, l_, n_tokens, s);
    if (rc) break;
  }
  if (sa != s) {   // join, also after an error
    cudaEvent_t e = h->ev_fork[h->ev_next++ % femto_handle::N_FORK];
    cudaEventRecord(e, sa);
    cudaStreamWaitEvent(s, e, 0);
  }
  if (rc) return rc;
  // every rank now holds the new values of the ranges it owns; fetch the others' (a handle without a
  // communicator skips this: the caller merges the ranges itself, as the single-GPU emulation test does)
  if (sharded && o->h->dp && o->exchange_mode == 1) {
    // The update kernels wrote this rank's share of the compute-type weights.  Clear the shares of the others and
    // add everybody's up: x + 0 + ... + 0 is exact in any type, and one large all-reduce is the collective NCCL
    // runs fastest.  The fp32 Theta of foreign ranges is NOT refreshed here (optimizer_gather_theta does that).
    for (size_t i = 0; i + 1 < o->foreign_weights.size(); i += 2)
      CUDA_TRY(cudaMemsetAsync(h->weights_begin + o->foreign_weights[i], 0, o->foreign_weights[i + 1], s));
    const long long n = (long long)((h->weights_end - h->weights_begin) / (h->bf ? 2 : 4));
    if (h->bf) FEMTO_TRY(dp_allreduce_sum_bf16(h->dp, h->weights_begin, n, s));
    else FEMTO_TRY(dp_allreduce_sum_f32(h->dp, reinterpret_cast<float*>(h->weights_begin), n, s));
    o->h->weights_valid = true;
    return 0;
  }
  if (sharded && o->h->dp) {
    for (size_t i = 0; i + 1 < o->foreign.size(); i += 2)
      CUDA_TRY(cudaMemsetAsync(theta + o->foreign[i], 0, sizeof(float) * (size_t)o->foreign[i + 1], s));
    FEMTO_TRY(dp_allreduce_sum_f32(o->h->dp, theta, o->h->nparams, s));   // x + 0 + ... + 0 is exact
    return model_refresh(o->h, theta, s);   // the ranges other ranks updated arrive as fp32 only
  }
  if (sharded) return model_refresh(o->h, theta, s);   // no communicator: the caller merges Theta and refreshes again
  // every weight the model reads in its compute type was rewritten by the update kernels above
  o->h->weights_valid = true;
  return 0;
}

int optimizer_get_t(femto_optimizer* o, int* t, int cap) {
  int n = (int)o->adam.size();
  for (int i = 0; i < n && i < cap; i++) t[i] = o->adam[i].t;
  return n;
}
int optimizer_set_t(femto_optimizer* o, const int* t, int count) {
  if (count != (int)o->adam.size()) return femto_fail(FEMTO_ERR_SHAPE, "expected %d step counters", (int)o->adam.size());
  for (int i = 0; i < count; i++) o->adam[i].t = t[i];
  return 0;
}

// Owner-sharded update for data parallelism.  Gradients are identical on every rank after the all-reduce, so
// instead of repeating the whole update on each of them, rank r updates only
//   * slice r of `world` equal slices of every large AdamW table (embeddings, lm_head, value embeddings), and
//   * the Muon matrices of the blocks [r L / world, (r+1) L / world),
// and the new values are exchanged: every rank clears the ranges it does not own and one all-reduce over Theta
// adds each owner's values to zeros (exact; NCCL's single large all-reduce is its fastest path, several times
// the rate of per-range all-gathers and broadcasts).  Small AdamW groups (scalars, gates) stay replicated.  The moments of ranges a rank does not own
// are not advanced on that rank: a checkpoint of the optimiser state has to collect every range from its owner.
int optimizer_set_shard(femto_optimizer* o, int rank, int world) {
  if (!o) return femto_fail(FEMTO_ERR_ARG, "NULL optimizer");
  if (world < 1 || rank < 0 || rank >= world) return femto_fail(FEMTO_ERR_ARG, "need 0 <= rank < world");
  femto_handle* h = o->h;
  if (world > 1 && h->dp && (dp_world(h->dp) != world || dp_rank(h->dp) != rank))
    return femto_fail(FEMTO_ERR_ARG, "rank / world differ from the handle's communicator (%d / %d)", dp_rank(h->dp),
                      dp_world(h->dp));
  o->shard_rank = rank; o->shard_world = world;
  o->gathers.clear(); o->bcasts.clear(); o->gaps.clear(); o->foreign.clear();
  for (auto& g : o->adam) {
    g.shard = world > 1 && g.n >= (1ll << 20) && g.n % (4ll * world) == 0;
    if (g.shard) { o->gathers.push_back(g.off); o->gathers.push_back(g.n / world); }
  }
  struct R { long long off, n; int owner; };
  std::vector<R> rs;
  const size_t es_model = h->bf ? 2 : 4;
  auto clear_w = [&](const void* ptr, size_t bytes) {
    if (!ptr || bytes == 0) return;
    const size_t off = (size_t)(reinterpret_cast<const char*>(ptr) - h->weights_begin);
    const size_t m = o->foreign_weights.size();
    if (m && o->foreign_weights[m - 2] + o->foreign_weights[m - 1] == off) o->foreign_weights[m - 1] += bytes;
    else { o->foreign_weights.push_back(off); o->foreign_weights.push_back(bytes); }
  };
  o->foreign_weights.clear();
  for (auto& g : o->muon) {
    const int k = (int)g.offs.size();
    g.k0 = 0; g.k1 = k;
    if (world == 1) continue;
    // the value-embedding gates (n_kv_head x 12) are read from Theta in fp32 by the forward pass and cost nothing
    // to update: every rank keeps updating all of them, like the scalars
    if ((long long)g.in * g.out < 1024) continue;
    g.k0 = k; g.k1 = k;
    for (int i = 0; i < k; i++) {
      const int owner = (int)((long long)g.layers[i] * world / h->L);
      if (owner == rank) { g.k0 = std::min(g.k0, i); g.k1 = i + 1; }
      rs.push_back({g.offs[i], (long long)g.in * g.out, owner});
    }
    if (g.k0 > g.k1) g.k0 = g.k1;
  }
  std::sort(rs.begin(), rs.end(), [](const R& a, const R& b) { return a.off < b.off; });
  for (size_t i = 0; i < rs.size(); i++) {
    const size_t m = o->bcasts.size();
    if (m && o->bcasts[m - 1] == rs[i].owner && o->bcasts[m - 3] + o->bcasts[m - 2] == rs[i].off) o->bcasts[m - 2] += rs[i].n;
    else { o->bcasts.push_back(rs[i].off); o->bcasts.push_back(rs[i].n); o->bcasts.push_back(rs[i].owner); }
  }
  // the replicated remainder of [0, nparams)
  std::vector<std::pair<long long, long long>> cover;
  for (size_t i = 0; i + 1 < o->gathers.size(); i += 2) cover.push_back({o->gathers[i], o->gathers[i + 1] * world});
  for (size_t i = 0; i + 2 < o->bcasts.size(); i += 3) cover.push_back({o->bcasts[i], o->bcasts[i + 1]});
  std::sort(cover.begin(), cover.end());
  long long at = 0;
  for (const auto& c : cover) {
    if (c.first > at) { o->gaps.push_back(at); o->gaps.push_back(c.first - at); }
    at = c.first + c.second;
  }
  if (world > 1 && at < h->nparams) { o->gaps.push_back(at); o->gaps.push_back(h->nparams - at); }
  // Exchange of Theta after the update: every rank clears what it does not own (the replicated gaps count as rank
  // 0's) and one all-reduce over the whole vector puts every range's new value, plus zeros, on every rank.
  auto clear = [&](long long off, long long n) {
    if (n <= 0) return;
    const size_t m = o->foreign.size();
    if (m && o->foreign[m - 2] + o->foreign[m - 1] == off) o->foreign[m - 1] += n;
    else { o->foreign.push_back(off); o->foreign.push_back(n); }
  };
  struct Q { long long off, n; int owner; };
  std::vector<Q> all;
  for (size_t i = 0; i + 1 < o->gathers.size(); i += 2)
    for (int r = 0; r < world; r++) all.push_back({o->gathers[i] + r * o->gathers[i + 1], o->gathers[i + 1], r});
  for (size_t i = 0; i + 2 < o->bcasts.size(); i += 3) all.push_back({o->bcasts[i], o->bcasts[i + 1], (int)o->bcasts[i + 2]});
  for (size_t i = 0; i + 1 < o->gaps.size(); i += 2) all.push_back({o->gaps[i], o->gaps[i + 1], 0});
  std::sort(all.begin(), all.end(), [](const Q& a, const Q& b) { return a.off < b.off; });
  for (const auto& q : all) if (q.owner != rank) clear(q.off, q.n);
  // the compute-type weights this rank does not write: foreign slices of the tables, every matrix of foreign blocks
  if (world > 1) {
    for (const auto& g : o->adam) {
      if (!g.shadow) continue;
      if (!g.shard) {
        // a table too small to slice is updated by every rank: in the exchange (a sum over ranks) it counts as rank 0's
        if (rank != 0) clear_w(g.shadow, (size_t)g.n * es_model);
        continue;
      }
      const size_t slice = (size_t)(g.n / world) * es_model;
      for (int r = 0; r < world; r++)
        if (r != rank) clear_w(reinterpret_cast<char*>(g.shadow) + (size_t)r * slice, slice);
    }
    for (int i = 0; i < h->L; i++) {
      if ((int)((long long)i * world / h->L) == rank) continue;
      const LayerBuf& l = h->lb[i];
      clear_w(l.sh_wqkv, es_model * (size_t)h->d * h->dq); clear_w(l.sh_wo, es_model * (size_t)h->d * h->d);
      clear_w(l.sh_fc, es_model * (size_t)4 * h->d * h->d); clear_w(l.sh_proj, es_model * (size_t)4 * h->d * h->d);
    }
    std::vector<std::pair<size_t, size_t>> fw;
    for (size_t i = 0; i + 1 < o->foreign_weights.size(); i += 2) fw.push_back({o->foreign_weights[i], o->foreign_weights[i + 1]});
    std::sort(fw.begin(), fw.end());
    o->foreign_weights.clear();
    for (const auto& q : fw) { o->foreign_weights.push_back(q.first); o->foreign_weights.push_back(q.second); }
  }
  return 0;
}

// How the owner-sharded update publishes its results.  mode 0 (default): the fp32 Theta is exchanged after every
// update, so the caller's parameter vector is complete on every rank at all times (what a single-GPU host expects).
// mode 1: only the model's compute-type weights are exchanged (half the bytes in a bf16 model, and no re-cast of
// Theta afterwards); the fp32 values of ranges owned elsewhere then lag behind until optimizer_gather_theta.
int optimizer_set_exchange(femto_optimizer* o, int mode) {
  if (!o || (mode != 0 && mode != 1)) return femto_fail(FEMTO_ERR_ARG, "mode must be 0 or 1");
  o->exchange_mode = mode;
  return 0;
}
// Completes the fp32 Theta on every rank: each rank clears what it does not own, one all-reduce adds the owners' values
// to zeros (exact).  Needed in exchange mode 1 before Theta is read by the host (checkpoint, evaluation elsewhere).
int optimizer_gather_theta(femto_optimizer* o, float* theta, cudaStream_t s) {
  if (!o || !theta) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  if (o->shard_world <= 1 || !o->h->dp) return 0;
  for (size_t i = 0; i + 1 < o->foreign.size(); i += 2)
    CUDA_TRY(cudaMemsetAsync(theta + o->foreign[i], 0, sizeof(float) * (size_t)o->foreign[i + 1], s));
  return dp_allreduce_sum_f32(o->h->dp, theta, o->h->nparams, s);
}
// Sum delta over ranks for this sharding: a range that one rank alone consumes is summed only onto that rank (on
// the others it keeps the local gradient), the rest is all-reduced.
int optimizer_grad_sync(femto_optimizer* o, float* delta, cudaStream_t s) {
  femto_handle* h = o->h;
  if (!h->dp) return 0;
  if (o->shard_world <= 1) return dp_allreduce_sum_f32(h->dp, delta, h->nparams, s);
  return dp_reduce_ranges(h->dp, delta, o->gathers.data(), (int)o->gathers.size() / 2, o->bcasts.data(),
                          (int)o->bcasts.size() / 3, o->gaps.data(), (int)o->gaps.size() / 2, s);
}
// (offset, count, owner) of every range that one rank alone updates; returns the number of triplets.
int optimizer_shard_ranges(femto_optimizer* o, long long* out, int cap) {
  int n = 0;
  auto put = [&](long long off, long long cnt, long long owner) {
    if (n < cap) { out[3 * n] = off; out[3 * n + 1] = cnt; out[3 * n + 2] = owner; }
    n++;
  };
  for (size_t i = 0; i + 1 < o->gathers.size(); i += 2)
    for (int r = 0; r < o->shard_world; r++) put(o->gathers[i] + r * o->gathers[i + 1], o->gathers[i + 1], r);
  for (size_t i = 0; i + 2 < o->bcasts.size(); i += 3) put(o->bcasts[i], o->bcasts[i + 1], o->bcasts[i + 2]);
  return n;
}
femto_handle* optimizer_handle(femto_optimizer* o) { return o->h; }

// Which rank holds the current moments of which part of a state buffer under the sharding (which: 0 adam_m,
// 1 adam_v, 2 muon_m, 3 muon_v): sorted (offset, count, owner) triplets covering the whole buffer.  Replicated
// groups are listed with owner 0 (every rank holds the same values).
static void state_cover(femto_optimizer* o, int which, std::vector<long long>& out) {
  const int world = o->shard_world, L = o->h->L;
  auto put = [&](long long off, long long n, long long owner) {
    const size_t m = out.size();
    if (m && out[m - 1] == owner && out[m - 3] + out[m - 2] == off) out[m - 2] += n;
    else { out.push_back(off); out.push_back(n); out.push_back(owner); }
  };
  if (which < 2) {
    for (const auto& g : o->adam) {
      if (g.shard) for (int r = 0; r < world; r++) put(g.moff + r * (g.n / world), g.n / world, r);
      else put(g.moff, g.n, 0);
    }
  } else {
    for (const auto& g : o->muon) {
      const long long per = which == 2 ? (long long)g.in * g.out : (long long)(g.out >= g.in ? g.out : g.in);
      const long long base = which == 2 ? g.moff : g.voff;
      for (size_t i = 0; i < g.offs.size(); i++)
        put(base + (long long)i * per, per,
            (world > 1 && (long long)g.in * g.out >= 1024) ? (long long)g.layers[i] * world / L : 0);   // gates: replicated
    }
  }
}
int optimizer_state_ranges(femto_optimizer* o, int which, long long* out, int cap) {
  if (which < 0 || which > 3) return femto_fail(FEMTO_ERR_ARG, "which must be 0..3");
  std::vector<long long> c;
  state_cover(o, which, c);
  const int n = (int)c.size() / 3;
  for (int i = 0; i < n && i < cap; i++) { out[3 * i] = c[3 * i]; out[3 * i + 1] = c[3 * i + 1]; out[3 * i + 2] = c[3 * i + 2]; }
  return n;
}
// Make the four state buffers complete on every rank (before a checkpoint, or before changing the sharding): each
// rank clears the parts whose current values live elsewhere and one all-reduce per buffer adds the owners' values
// to zeros (src/checkpoints.jl:9-12 reads the moments group by group from one process).
int optimizer_gather_state(femto_optimizer* o, cudaStream_t s) {
  femto_handle* h = o->h;
  if (o->shard_world <= 1 || !h->dp) return 0;
  long long sizes[4];
  FEMTO_TRY(optimizer_state_sizes(h, sizes));
  float* bufs[4] = {o->adam_m, o->adam_v, o->muon_m, o->muon_v};
  for (int w = 0; w < 4; w++) {
    std::vector<long long> c;
    state_cover(o, w, c);
    for (size_t i = 0; i + 2 < c.size(); i += 3)
      if (c[i + 2] != o->shard_rank) CUDA_TRY(cudaMemsetAsync(bufs[w] + c[i], 0, sizeof(float) * (size_t)c[i + 1], s));
    FEMTO_TRY(dp_allreduce_sum_f32(h->dp, bufs[w], sizes[w], s));
  }
  return 0;
}
