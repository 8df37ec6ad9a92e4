// Host wrappers of the HBM-streaming kernels (norms, residual mixes, RoPE + QK-norm, smear,
// gates, casts).  T is the activation type (float or bf16); statistics and parameters are fp32.
#pragma once
#include "common.cuh"

template <typename T> struct Stream {
  static int prep_tokens(const int* tokens, const int* targets, const int* positions, int B, int Tlen,
                         int index_base, int vocab, int maxdoc, int* tok0, int* tgt0, int* pos, int* doc_start,
                         unsigned int* status, cudaStream_t s);
  static int embed_norm(const T* table, const int* tok0, T* xe, int N, int D, float eps, cudaStream_t s);
  static int smear(const T* xe, const float* w_s, const float* lam_s, int N, int Tlen, int D, float* sg, T* x0,
                   cudaStream_t s);
  static int mix_norm(const T* xin, const T* x0, const float* lam_b, const float* lam_x0, T* xm, T* xn, float* r,
                      int N, int D, float eps, cudaStream_t s);
  static int norm(const T* x, T* xn, float* r, int N, int D, float eps, cudaStream_t s);
  static int qkv_post(T* qkv, long long ldq, const T* xn1, int D, const float* ve_gate, const T* ve_table,
                      const int* tok0, const int* pos, const float* sin_t, const float* cos_t, int N, int H,
                      int Hkv, int hd, float eps, float* rqk, float* sv, cudaStream_t s);
  static int qkv_post_bwd(T* dqkv, const T* qkv, long long ldq, const T* ve_table, const int* tok0,
                          const int* pos, const float* sin_t, const float* cos_t, int N, int H, int Hkv, int hd,
                          const float* rqk, const float* sv, T* dve, float* dpre, cudaStream_t s);
  static int ve_gate_bwd(const T* xn1, int D, const float* dpre, const float* ve_gate, T* dxn, int N, int Hkv,
                         float* partial, int* nblocks_out, cudaStream_t s);
  static int norm_bwd_resid(const T* dy, const T* y, const float* r, const T* resid, T* out, int N, int D,
                            cudaStream_t s);
  static int mix_bwd(const T* dx_in, T* dx, const T* dxn, const T* xn1, const float* r1, const T* xin, const T* x0,
                     const float* lam_b, const float* lam_x0, T* dx0, bool first, int N, int D, float* partial,
                     int* nblocks_out, cudaStream_t s);
  static int backout_norm(const T* xl, const T* xb, const float* lam_y, T* xf_scratch, T* xnf, float* rf, int N,
                          int D, float eps, cudaStream_t s);
  static int head_bwd(const T* dxnf, const T* xnf, const float* rf, const T* xb, T* dxf, int N, int D,
                      float* partial, int* nblocks_out, cudaStream_t s);
  static int axpy(T* y, const T* x, const float* a_dev, float a_mul, long long n, cudaStream_t s);
  static int add(T* y, const T* x, long long n, cudaStream_t s);
  static int smear_gate_bwd(const T* dx0, const T* xe, const float* sg, const float* lam_s, int N, int Tlen,
                            int D, float* dpre, float* partial, int* nblocks_out, cudaStream_t s);
  static int embed_bwd(const T* dx0, const T* table, const int* tok0, const T* xe, const float* sg,
                       const float* dpre, const float* w_s, const float* lam_s, int N, int Tlen, int D,
                       float eps, T* dE, cudaStream_t s);
  static int xent_rows(const float* logits, long long ldl, const int* tgt0, int n, int V, float w,
                       const float* w_dev, T* dlogit,
                       long long lddl, float* loss_rows, cudaStream_t s);
  static int cast_from_f32(const float* src, T* dst, long long n, cudaStream_t s);
  static int pack_qkv(const float* wq, const float* wk, const float* wv, T* dst, int D, int kv, cudaStream_t s);
};

int sum_rows_to_scalar(const float* rows, int n, float* out, const int* tgt0, int* n_valid_out, float scale_by_valid,
                       cudaStream_t s);
int xent_dlogit_inplace(void* logits_bf16, long long ld, const float* lse_rows, const int* tgt0, int n, int V, float w,
                        const float* w_dev, cudaStream_t s);
int softcap_inplace(float* x, long long n, cudaStream_t s);
int xent_finalize(const float2* stats, int ntile, const float* tz, const int* tgt0, int n, float* lse,
                  float* loss_rows, cudaStream_t s);
int fill_zero(void* p, size_t bytes, cudaStream_t s);
