// The handle behind the C ABI: configuration, flat layout, workspace arena and the
// forward / reverse schedule of the GPT step.
#pragma once
#include <string>
#include <vector>

#include "common.cuh"

struct LayerP {
  long long wq, wk, wv, wo, ve_gate, fc, proj, ve_table, lam_b, lam_x0;  // element offsets into Theta
  bool ve;
  int window;  // left window (keys t-window..t)
};

struct LayerBuf {
  void *sh_wqkv = nullptr, *sh_wo = nullptr, *sh_fc = nullptr, *sh_proj = nullptr, *sh_ve = nullptr;  // weights, type T
  void *xout = nullptr, *xn1 = nullptr, *qkv = nullptr, *att = nullptr, *xn2 = nullptr, *a = nullptr;   // saved activations
  float *r1 = nullptr, *r2 = nullptr, *rqk = nullptr, *sv = nullptr, *lse = nullptr;
};

struct DpState;  // NCCL communicator (dp.cu)

struct femto_handle {
  femto_config cfg;
  int d = 0, H = 0, Hkv = 0, hd = 0, kv = 0, dq = 0, V = 0, Vp = 0, L = 0, T = 0, maxB = 0, maxN = 0;
  long long nparams = 0;
  float eps = 0.f;
  bool bf = false;
  std::vector<LayerP> lp;
  long long off_wte = 0, off_lm = 0, off_smear = 0, off_lam_s = 0, off_lam_y = 0;
  int backout = 0;  // 0-based index of the block whose output is subtracted before the head
  int rank = 0, world = 1;
  int xchunk = 0;   // tokens per lm_head-tail chunk

  char* arena = nullptr;
  size_t arena_bytes = 0;
  float *sin_t = nullptr, *cos_t = nullptr;
  unsigned int* status = nullptr;
  void *sh_wte = nullptr, *sh_lm = nullptr;
  char *weights_begin = nullptr, *weights_end = nullptr;   // the contiguous range holding every compute-type weight
  bool weights_valid = false;
  int *tok0 = nullptr, *tgt0 = nullptr, *pos = nullptr, *doc_start = nullptr, *raw_tok = nullptr, *raw_tgt = nullptr,
      *raw_pos = nullptr;
  void *xe = nullptr, *x0 = nullptr, *xm = nullptr, *xnf = nullptr;
  float *sg = nullptr, *rf = nullptr;
  std::vector<LayerBuf> lb;
  void *dx = nullptr, *dxn = nullptr, *dqkv = nullptr, *datt = nullptr, *du = nullptr, *dx0 = nullptr, *dxf = nullptr,
       *dve = nullptr;
  float *dpre = nullptr, *dpre_s = nullptr, *partial = nullptr;
  float* logits_f32 = nullptr;  // [xchunk][Vp], fp32 build / SIMT path only
  float2* xstats = nullptr;     // [xchunk][ceil(V/256)], tensor-core path
  float *tz = nullptr, *lse_rows = nullptr, *loss_rows = nullptr, *inv_nvalid = nullptr;
  void* dlogit = nullptr;       // [xchunk][Vp] of T
  float* loss_dev = nullptr;
  int* nvalid_dev = nullptr;
  void* gemm_ws = nullptr;
  size_t gemm_ws_bytes = 0;
  // Two internal streams for the training step: `hi` (highest priority) carries the dependency chain of the
  // forward and reverse pass, `lo` (lowest priority) the weight-gradient GEMMs, the zero fill of delta and the
  // AdamW tables of the update.  Nothing on the chain waits for that work within a block, so it fills the tensor
  // pipe while the chain runs its HBM-streaming kernels.  The caller's stream is joined on both sides of a call.
  cudaStream_t hi = nullptr, lo = nullptr;
  static constexpr int N_FORK = 16, N_SIDE = 12;
  cudaEvent_t ev_fork[N_FORK] = {};   // chain -> side, used round-robin (a wait keeps the record it was given)
  int ev_next = 0;
  cudaEvent_t ev_side[N_SIDE] = {};   // side -> chain: the last side reader of a gradient buffer has finished
  bool side_armed[N_SIDE] = {};
  void* gemm_ws2 = nullptr;           // split-K partials of the side stream's GEMMs
  void *dx_b = nullptr, *dx_c = nullptr, *du_b = nullptr, *dqkv_b = nullptr, *dlogit_b = nullptr;  // rotation partners
  void* attn_ws = nullptr;
  size_t attn_ws_bytes = 0;
  struct ScatterPlan* plan = nullptr;
  DpState* dp = nullptr;
  bool overlap_sync = false;     // sum delta over ranks in buckets while the reverse pass runs
  bool delta_synced = false;     // the last step already reduced delta (femto_grad_sync only joins)
  std::string err;
};

// Options of a forward pass that is not a training step: a sequence length other than the configured one (a
// prompt) and a key/value cache that takes the prompt's keys and values (decode.cu).
struct femto_kv_cache;
struct StepExtra {
  int T = 0;                        // rows per column of this call (0 = sequence_len)
  femto_kv_cache* cache = nullptr;  // filled from the prompt when set
  float* last_logits = nullptr;     // fp32 [B][vocab_size]: soft-capped logits of each column's last position
};
template <typename T> int kv_cache_store_prompt(femto_kv_cache* c, int B, int Tp, cudaStream_t s);
template <typename T> int kv_cache_last_logits(femto_kv_cache* c, const T* xnf, int B, int Tp, float* logits_out, cudaStream_t s);

int model_fill(femto_handle* h, const femto_config* cfg);  // derived sizes + layout, no device work
int model_alloc(femto_handle* h);
void model_free(femto_handle* h);
int model_refresh(femto_handle* h, const float* theta, cudaStream_t s);
int model_step(femto_handle* h, const float* theta, float* delta, const int* tokens, const int* targets,
               const int* positions, int B, int reduction, bool backward, bool accumulate, float* loss_out,
               int* nvalid_out, cudaStream_t s, float* logits_out = nullptr, float* token_losses_out = nullptr,
               const StepExtra* ex = nullptr);
int layout_describe(const femto_config* cfg, std::vector<femto_tensor_desc>& out, long long* nparams, int* Vp);
int layout_windows(const femto_config* cfg, std::vector<int>& left, std::vector<int>& has_ve);

int dp_create(DpState** out, int rank, int world, const void* id128);
void dp_destroy(DpState* d);
int dp_unique_id(void* id128);
int dp_allreduce_sum_f32(DpState* d, float* buf, long long n, cudaStream_t s);
int dp_allreduce_sum_i32(DpState* d, int* buf, long long n, cudaStream_t s);
int dp_allreduce_sum_bf16(DpState* d, void* buf, long long n, cudaStream_t s);
int dp_bucket_allreduce(DpState* d, float* buf, long long n, cudaStream_t compute);
int dp_join(DpState* d, cudaStream_t compute);
int dp_reduce_ranges(DpState* d, float* delta, const long long* gathers, int n_gathers, const long long* bcasts,
                     int n_bcasts, const long long* gaps, int n_gaps, cudaStream_t s);
int dp_async_error(DpState* d);
int dp_abort(DpState* d);
int dp_world(const DpState* d);
int dp_rank(const DpState* d);
