// Strided SIMT GEMM with fp32 accumulation.  It is the matrix multiply of the fp32 build
// (the reference's Float32 path, src/gpt.jl:23-31) and of shapes the tcgen05 kernel does not
// take (row pitches that are not multiples of 16 bytes, e.g. the 12 -> n_kv_head gate).
#include "common.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(GemmArgs g) {
  __shared__ float As[TK][TM + 1];
  __shared__ float Bs[TK][TN + 1];
  const int bz = blockIdx.z;
  const T* A = reinterpret_cast<const T*>(g.A) + (long long)bz * g.strideA;
  const T* B = reinterpret_cast<const T*>(g.B) + (long long)bz * g.strideB;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < g.K; k0 += TK) {
    // 64x16 elements of each operand, 4 per thread
#pragma unroll
    for (int e = 0; e < 4; e++) {
      int idx = tid + e * 256;
      int mm, kk;
      if (g.a_kmajor) { kk = idx % TK; mm = idx / TK; } else { mm = idx % TM; kk = idx / TM; }
      int gm = m0 + mm, gk = k0 + kk;
      float v = 0.f;
      if (gm < g.M && gk < g.K)
        v = to_f<T>(g.a_kmajor ? A[(long long)gm * g.lda + gk] : A[(long long)gk * g.lda + gm]);
      As[kk][mm] = v;
      int nn;
      if (g.b_kmajor) { kk = idx % TK; nn = idx / TK; } else { nn = idx % TN; kk = idx / TN; }
      int gn = n0 + nn;
      gk = k0 + kk;
      v = 0.f;
      if (gn < g.N && gk < g.K)
        v = to_f<T>(g.b_kmajor ? B[(long long)gn * g.ldb + gk] : B[(long long)gk * g.ldb + gn]);
      Bs[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; kk++) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

  T* C = reinterpret_cast<T*>(g.C) + (long long)bz * g.strideC;
  float* Cf = reinterpret_cast<float*>(g.C) + (long long)bz * g.strideC;
  const T* aux = reinterpret_cast<const T*>(g.aux) + (long long)bz * g.strideAux;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    int m = m0 + ty * 4 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int n = n0 + tx * 4 + j;
      if (n >= g.N) continue;
      float v = acc[i][j];
      switch (g.epi) {
        case EPI_STORE: C[(long long)m * g.ldc + n] = from_f<T>(v); break;
        case EPI_RESID:
          C[(long long)m * g.ldc + n] = from_f<T>(to_f<T>(aux[(long long)m * g.ldaux + n]) + v);
          break;
        case EPI_RELU2: { float r = fmaxf(v, 0.f); C[(long long)m * g.ldc + n] = from_f<T>(r * r); } break;
        case EPI_DRELU2:
          C[(long long)m * g.ldc + n] =
              from_f<T>(v * 2.f * sqrtf(fmaxf(to_f<T>(aux[(long long)m * g.ldaux + n]), 0.f)));
          break;
        case EPI_AXPBY:
          C[(long long)m * g.ldc + n] =
              from_f<T>(g.alpha * to_f<T>(aux[(long long)m * g.ldaux + n]) + g.beta * v);
          break;
        case EPI_F32: {
          float* dst;
          if (g.nseg == 0) {
            dst = Cf + (long long)m * g.ldc + n;
          } else {
            dst = nullptr;
            for (int s = 0; s < g.nseg; s++)
              if (n >= g.seg_col0[s] && n < g.seg_col0[s] + g.seg_ncol[s])
                dst = g.seg_ptr[s] + (long long)m * g.seg_ld[s] + (n - g.seg_col0[s]);
            if (!dst) break;
          }
          *dst = (g.beta != 0.f ? *dst : 0.f) + g.alpha * v;
        } break;
        default: break;
      }
    }
  }
}

}  // namespace

template <typename T> int gemm_simt(const GemmArgs& g, cudaStream_t s) {
  if (g.epi > EPI_F32) return femto_fail(FEMTO_ERR_UNSUPPORTED, "gemm_simt: epilogue %d needs the tensor-core path", g.epi);
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return femto_fail(FEMTO_ERR_SHAPE, "gemm_simt: empty problem");
  dim3 grid(cdiv(g.N, TN), cdiv(g.M, TM), g.batch);
  gemm_simt_kernel<T><<<grid, 256, 0, s>>>(g);
  KERNEL_CHECK();
  return 0;
}
template int gemm_simt<float>(const GemmArgs&, cudaStream_t);
template int gemm_simt<bf16>(const GemmArgs&, cudaStream_t);

template <> int gemm<float>(const GemmArgs& g, cudaStream_t s) { return gemm_simt<float>(g, s); }
template <> int gemm<bf16>(const GemmArgs& g, cudaStream_t s) {
  if (gemm_tc_supported(g)) return gemm_tc_bf16(g, s);
  return gemm_simt<bf16>(g, s);
}
