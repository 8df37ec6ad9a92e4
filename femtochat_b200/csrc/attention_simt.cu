// Plain SIMT attention (forward and reverse) for any head_dim <= 256 and any dtype.  It serves
// the fp32 build (the reference's Float32 path, src/kernels.jl:131-219,287-379) and head sizes
// the tcgen05 kernels do not take.  One warp owns one output row, keys are visited in order, so
// results are deterministic.  Mask: key k is visible to query t iff t-left <= k <= t
// (src/kernels.jl:38) and, with doc_start, k >= doc_start[t].
#include "common.cuh"

namespace {

constexpr int EPL = 8;  // elements per lane: head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(128) attn_fwd_simt_kernel(AttnArgs a) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int t = blockIdx.x * 4 + warp, h = blockIdx.y, b = blockIdx.z;
  if (t >= a.T) return;
  const int kvh = h / (a.H / a.Hkv);
  const int hd = a.hd;
  const float scale = rsqrtf((float)hd);
  const T* q = reinterpret_cast<const T*>(a.Q) + ((long long)b * a.T + t) * a.q_stride + (long long)h * hd;
  float qv[EPL], acc[EPL];
#pragma unroll
  for (int e = 0; e < EPL; e++) {
    int d = lane + 32 * e;
    qv[e] = d < hd ? to_f<T>(q[d]) : 0.f;
    acc[e] = 0.f;
  }
  int k0 = max(0, t - a.window_left);
  if (a.doc_start) k0 = max(k0, a.doc_start[(long long)b * a.T + t]);
  float m = -INFINITY, l = 0.f;
  for (int k = k0; k <= t; k++) {
    const T* kp = reinterpret_cast<const T*>(a.K) + ((long long)b * a.T + k) * a.kv_stride + (long long)kvh * hd;
    const T* vp = reinterpret_cast<const T*>(a.V) + ((long long)b * a.T + k) * a.kv_stride + (long long)kvh * hd;
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; e++) {
      int d = lane + 32 * e;
      if (d < hd) s = fmaf(qv[e], to_f<T>(kp[d]), s);
    }
    s = warp_sum(s) * scale;
    float mn = fmaxf(m, s);
    float alpha = expf(m - mn), p = expf(s - mn);
    l = l * alpha + p;
#pragma unroll
    for (int e = 0; e < EPL; e++) {
      int d = lane + 32 * e;
      if (d < hd) acc[e] = acc[e] * alpha + p * to_f<T>(vp[d]);
    }
    m = mn;
  }
  T* o = reinterpret_cast<T*>(a.O) + ((long long)b * a.T + t) * a.o_stride + (long long)h * hd;
  float inv = 1.f / l;
#pragma unroll
  for (int e = 0; e < EPL; e++) {
    int d = lane + 32 * e;
    if (d < hd) o[d] = from_f<T>(acc[e] * inv);
  }
  if (lane == 0) {
    long long si = ((long long)b * a.H + h) * a.T + t;
    if (a.lse) a.lse[si] = m + logf(l);
    if (a.l) a.l[si] = l;
    if (a.m) a.m[si] = m;
  }
}

// dQ and the row term D = sum(dO*O): one warp per (b, h, query).
template <typename T>
__global__ void __launch_bounds__(128) attn_bwd_dq_simt_kernel(AttnArgs a, float* Dbuf) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int t = blockIdx.x * 4 + warp, h = blockIdx.y, b = blockIdx.z;
  if (t >= a.T) return;
  const int kvh = h / (a.H / a.Hkv);
  const int hd = a.hd;
  const float scale = rsqrtf((float)hd);
  const long long row = (long long)b * a.T + t;
  const T* q = reinterpret_cast<const T*>(a.Q) + row * a.q_stride + (long long)h * hd;
  const T* o = reinterpret_cast<const T*>(a.O) + row * a.o_stride + (long long)h * hd;
  const T* dO = reinterpret_cast<const T*>(a.dO) + row * a.do_stride + (long long)h * hd;
  float qv[EPL], dov[EPL], acc[EPL];
  float D = 0.f;
#pragma unroll
  for (int e = 0; e < EPL; e++) {
    int d = lane + 32 * e;
    qv[e] = d < hd ? to_f<T>(q[d]) : 0.f;
    dov[e] = d < hd ? to_f<T>(dO[d]) : 0.f;
    D += d < hd ? dov[e] * to_f<T>(o[d]) : 0.f;
    acc[e] = 0.f;
  }
  D = warp_sum(D);
  const long long si = ((long long)b * a.H + h) * a.T + t;
  if (lane == 0) Dbuf[si] = D;
  const float lse = a.lse[si];
  int k0 = max(0, t - a.window_left);
  if (a.doc_start) k0 = max(k0, a.doc_start[row]);
  for (int k = k0; k <= t; k++) {
    const T* kp = reinterpret_cast<const T*>(a.K) + ((long long)b * a.T + k) * a.kv_stride + (long long)kvh * hd;
    const T* vp = reinterpret_cast<const T*>(a.V) + ((long long)b * a.T + k) * a.kv_stride + (long long)kvh * hd;
    float s = 0.f, dp = 0.f;
    float kv[EPL];
#pragma unroll
    for (int e = 0; e < EPL; e++) {
      int d = lane + 32 * e;
      kv[e] = d < hd ? to_f<T>(kp[d]) : 0.f;
      s = fmaf(qv[e], kv[e], s);
      if (d < hd) dp = fmaf(dov[e], to_f<T>(vp[d]), dp);
    }
    s = warp_sum(s) * scale;
    dp = warp_sum(dp);
    float p = expf(s - lse);
    float ds = p * (dp - D) * scale;
#pragma unroll
    for (int e = 0; e < EPL; e++) acc[e] = fmaf(ds, kv[e], acc[e]);
  }
  T* dq = reinterpret_cast<T*>(a.dQ) + row * a.dq_stride + (long long)h * hd;
#pragma unroll
  for (int e = 0; e < EPL; e++) {
    int d = lane + 32 * e;
    if (d < hd) dq[d] = from_f<T>(a.accumulate ? to_f<T>(dq[d]) + acc[e] : acc[e]);
  }
}

// dK, dV: one warp per (b, kv head, key); loops over the heads of the GQA group and the queries
// that see this key, in order.
template <typename T>
__global__ void __launch_bounds__(128) attn_bwd_dkv_simt_kernel(AttnArgs a, const float* Dbuf) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int k = blockIdx.x * 4 + warp, kvh = blockIdx.y, b = blockIdx.z;
  if (k >= a.T) return;
  const int g = a.H / a.Hkv;
  const int hd = a.hd;
  const float scale = rsqrtf((float)hd);
  const long long krow = (long long)b * a.T + k;
  const T* kp = reinterpret_cast<const T*>(a.K) + krow * a.kv_stride + (long long)kvh * hd;
  const T* vp = reinterpret_cast<const T*>(a.V) + krow * a.kv_stride + (long long)kvh * hd;
  float kv[EPL], vv[EPL], dk[EPL], dv[EPL];
#pragma unroll
  for (int e = 0; e < EPL; e++) {
    int d = lane + 32 * e;
    kv[e] = d < hd ? to_f<T>(kp[d]) : 0.f;
    vv[e] = d < hd ? to_f<T>(vp[d]) : 0.f;
    dk[e] = 0.f;
    dv[e] = 0.f;
  }
  const long long t1 = min((long long)a.T - 1, (long long)k + a.window_left);
  for (int hh = 0; hh < g; hh++) {
    const int h = kvh * g + hh;
    for (int t = k; t <= t1; t++) {
      const long long row = (long long)b * a.T + t;
      if (a.doc_start && a.doc_start[row] > k) continue;
      const T* q = reinterpret_cast<const T*>(a.Q) + row * a.q_stride + (long long)h * hd;
      const T* dO = reinterpret_cast<const T*>(a.dO) + row * a.do_stride + (long long)h * hd;
      float qv[EPL], dov[EPL];
      float s = 0.f, dp = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; e++) {
        int d = lane + 32 * e;
        qv[e] = d < hd ? to_f<T>(q[d]) : 0.f;
        dov[e] = d < hd ? to_f<T>(dO[d]) : 0.f;
        s = fmaf(qv[e], kv[e], s);
        dp = fmaf(dov[e], vv[e], dp);
      }
      s = warp_sum(s) * scale;
      dp = warp_sum(dp);
      const long long si = ((long long)b * a.H + h) * a.T + t;
      float p = expf(s - a.lse[si]);
      float ds = p * (dp - Dbuf[si]) * scale;
#pragma unroll
      for (int e = 0; e < EPL; e++) {
        dk[e] = fmaf(ds, qv[e], dk[e]);
        dv[e] = fmaf(p, dov[e], dv[e]);
      }
    }
  }
  T* dkp = reinterpret_cast<T*>(a.dK) + krow * a.dkv_stride + (long long)kvh * hd;
  T* dvp = reinterpret_cast<T*>(a.dV) + krow * a.dkv_stride + (long long)kvh * hd;
#pragma unroll
  for (int e = 0; e < EPL; e++) {
    int d = lane + 32 * e;
    if (d < hd) {
      dkp[d] = from_f<T>(a.accumulate ? to_f<T>(dkp[d]) + dk[e] : dk[e]);
      dvp[d] = from_f<T>(a.accumulate ? to_f<T>(dvp[d]) + dv[e] : dv[e]);
    }
  }
}

}  // namespace

template <typename T> int attention_fwd_simt(const AttnArgs& a, cudaStream_t s) {
  if (a.hd > 32 * EPL) return femto_fail(FEMTO_ERR_UNSUPPORTED, "attention: head_dim %d > %d", a.hd, 32 * EPL);
  dim3 grid(cdiv(a.T, 4), a.H, a.B);
  attn_fwd_simt_kernel<T><<<grid, 128, 0, s>>>(a);
  KERNEL_CHECK();
  return 0;
}
template <typename T> int attention_bwd_simt(const AttnArgs& a, cudaStream_t s) {
  if (a.hd > 32 * EPL) return femto_fail(FEMTO_ERR_UNSUPPORTED, "attention: head_dim %d > %d", a.hd, 32 * EPL);
  size_t need = sizeof(float) * (size_t)a.B * a.H * a.T;
  if (!a.ws || a.ws_bytes < need) return femto_fail(FEMTO_ERR_ARG, "attention_bwd: workspace too small");
  float* D = reinterpret_cast<float*>(a.ws);
  dim3 grid(cdiv(a.T, 4), a.H, a.B);
  attn_bwd_dq_simt_kernel<T><<<grid, 128, 0, s>>>(a, D);
  KERNEL_CHECK();
  dim3 grid2(cdiv(a.T, 4), a.Hkv, a.B);
  attn_bwd_dkv_simt_kernel<T><<<grid2, 128, 0, s>>>(a, D);
  KERNEL_CHECK();
  return 0;
}
template int attention_fwd_simt<float>(const AttnArgs&, cudaStream_t);
template int attention_fwd_simt<bf16>(const AttnArgs&, cudaStream_t);
template int attention_bwd_simt<float>(const AttnArgs&, cudaStream_t);
template int attention_bwd_simt<bf16>(const AttnArgs&, cudaStream_t);

template <> int attention_fwd<float>(const AttnArgs& a, cudaStream_t s) { return attention_fwd_simt<float>(a, s); }
template <> int attention_bwd<float>(const AttnArgs& a, cudaStream_t s) { return attention_bwd_simt<float>(a, s); }
template <> int attention_fwd<bf16>(const AttnArgs& a, cudaStream_t s) {
  if (attention_tc_supported(a)) return attention_fwd_tc(a, s);
  return attention_fwd_simt<bf16>(a, s);
}
template <> int attention_bwd<bf16>(const AttnArgs& a, cudaStream_t s) {
  if (attention_tc_supported(a)) return attention_bwd_tc(a, s);
  return attention_bwd_simt<bf16>(a, s);
}
