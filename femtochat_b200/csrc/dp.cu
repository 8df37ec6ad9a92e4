// Data-parallel plumbing: one NCCL communicator per handle.  The reference has no distributed
// path at all (scripts/train.jl:13 "Single-GPU base training"); this layer is new.  NCCL is
// resolved at run time with dlopen so the library loads (and the layout / host entry points work)
// on machines without it; a data-parallel call without NCCL fails with a clear error.
#include <dlfcn.h>
#include <string.h>

#include "model.cuh"

namespace {
typedef struct { char internal[128]; } nccl_uid;
typedef void* nccl_comm;
typedef int (*fn_get_uid)(nccl_uid*);
typedef int (*fn_init_rank)(nccl_comm*, int, nccl_uid, int);
typedef int (*fn_destroy)(nccl_comm);
typedef int (*fn_allreduce)(const void*, void*, size_t, int, int, nccl_comm, cudaStream_t);
typedef int (*fn_reduce_scatter)(const void*, void*, size_t, int, int, nccl_comm, cudaStream_t);
typedef int (*fn_reduce)(const void*, void*, size_t, int, int, int, nccl_comm, cudaStream_t);
typedef int (*fn_group)(void);
typedef const char* (*fn_errstr)(int);
typedef int (*fn_async_err)(nccl_comm, int*);
typedef int (*fn_abort)(nccl_comm);

struct Nccl {
  void* lib = nullptr;
  fn_get_uid get_uid = nullptr; fn_init_rank init_rank = nullptr; fn_destroy destroy = nullptr;
  fn_allreduce allreduce = nullptr; fn_reduce_scatter reduce_scatter = nullptr;
  fn_reduce reduce = nullptr; fn_group group_start = nullptr, group_end = nullptr;
  fn_errstr errstr = nullptr;
  fn_async_err async_err = nullptr; fn_abort abort = nullptr;
};
Nccl g_nccl;

int nccl_load() {
  if (g_nccl.lib) return 0;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    g_nccl.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (g_nccl.lib) break;
  }
  if (!g_nccl.lib) return femto_fail(FEMTO_ERR_UNSUPPORTED, "libnccl.so.2 not found: %s", dlerror());
  g_nccl.get_uid = (fn_get_uid)dlsym(g_nccl.lib, "ncclGetUniqueId");
  g_nccl.init_rank = (fn_init_rank)dlsym(g_nccl.lib, "ncclCommInitRank");
  g_nccl.destroy = (fn_destroy)dlsym(g_nccl.lib, "ncclCommDestroy");
  g_nccl.allreduce = (fn_allreduce)dlsym(g_nccl.lib, "ncclAllReduce");
  g_nccl.reduce_scatter = (fn_reduce_scatter)dlsym(g_nccl.lib, "ncclReduceScatter");
  g_nccl.reduce = (fn_reduce)dlsym(g_nccl.lib, "ncclReduce");
  g_nccl.group_start = (fn_group)dlsym(g_nccl.lib, "ncclGroupStart");
  g_nccl.group_end = (fn_group)dlsym(g_nccl.lib, "ncclGroupEnd");
  g_nccl.errstr = (fn_errstr)dlsym(g_nccl.lib, "ncclGetErrorString");
  g_nccl.async_err = (fn_async_err)dlsym(g_nccl.lib, "ncclCommGetAsyncError");
  g_nccl.abort = (fn_abort)dlsym(g_nccl.lib, "ncclCommAbort");
  if (!g_nccl.get_uid || !g_nccl.init_rank || !g_nccl.allreduce || !g_nccl.reduce_scatter ||
      !g_nccl.reduce || !g_nccl.group_start || !g_nccl.group_end)
    return femto_fail(FEMTO_ERR_UNSUPPORTED, "libnccl is missing required symbols");
  return 0;
}
// ncclDataType_t / ncclRedOp_t values of the public nccl.h
constexpr int NCCL_INT32 = 2, NCCL_FLOAT32 = 7, NCCL_BFLOAT16 = 9, NCCL_SUM = 0;
int nccl_check(int r, const char* what) {
  if (r == 0) return 0;
  return femto_fail(200000 + r, "%s failed: %s", what, g_nccl.errstr ? g_nccl.errstr(r) : "nccl error");
}
}  // namespace

struct DpState {
  nccl_comm comm = nullptr;
  int rank = 0, world = 1;
  cudaStream_t cs = nullptr;      // communication stream: bucket all-reduces overlap the reverse pass
  cudaEvent_t ready = nullptr;    // compute -> comm: the bucket's gradients are complete
  cudaEvent_t done = nullptr;     // comm -> compute: every queued bucket has been reduced
  bool pending = false;
};

int dp_unique_id(void* id128) {
  FEMTO_TRY(nccl_load());
  nccl_uid id;
  FEMTO_TRY(nccl_check(g_nccl.get_uid(&id), "ncclGetUniqueId"));
  memcpy(id128, &id, 128);
  return 0;
}

int dp_create(DpState** out, int rank, int world, const void* id128) {
  if (world <= 1) { *out = nullptr; return 0; }
  if (!id128) return femto_fail(FEMTO_ERR_ARG, "world > 1 needs the shared ncclUniqueId");
  FEMTO_TRY(nccl_load());
  DpState* d = new DpState();
  d->rank = rank; d->world = world;
  nccl_uid id;
  memcpy(&id, id128, 128);
  int r = nccl_check(g_nccl.init_rank(&d->comm, world, id, rank), "ncclCommInitRank");
  if (r) { delete d; return r; }
  CUDA_TRY(cudaStreamCreateWithFlags(&d->cs, cudaStreamNonBlocking));
  CUDA_TRY(cudaEventCreateWithFlags(&d->ready, cudaEventDisableTiming));
  CUDA_TRY(cudaEventCreateWithFlags(&d->done, cudaEventDisableTiming));
  *out = d;
  return 0;
}

// Queue an in-place sum over ranks of buf[0..n) on the communication stream, ordered after
// everything already enqueued on `compute`.
int dp_bucket_allreduce(DpState* d, float* buf, long long n, cudaStream_t compute) {
  if (!d || n <= 0) return 0;
  if (!d->comm) return femto_fail(FEMTO_ERR_STATE, "the communicator was aborted");
  CUDA_TRY(cudaEventRecord(d->ready, compute));
  CUDA_TRY(cudaStreamWaitEvent(d->cs, d->ready, 0));
  FEMTO_TRY(nccl_check(g_nccl.allreduce(buf, buf, (size_t)n, NCCL_FLOAT32, NCCL_SUM, d->comm, d->cs), "ncclAllReduce"));
  d->pending = true;
  return 0;
}
// Make `compute` wait for every queued bucket.
int dp_join(DpState* d, cudaStream_t compute) {
  if (!d || !d->pending) return 0;
  CUDA_TRY(cudaEventRecord(d->done, d->cs));
  CUDA_TRY(cudaStreamWaitEvent(compute, d->done, 0));
  d->pending = false;
  return 0;
}

void dp_destroy(DpState* d) {
  if (!d) return;
  if (d->cs) cudaStreamSynchronize(d->cs);
  if (d->comm && g_nccl.destroy) g_nccl.destroy(d->comm);
  if (d->ready) cudaEventDestroy(d->ready);
  if (d->done) cudaEventDestroy(d->done);
  if (d->cs) cudaStreamDestroy(d->cs);
  delete d;
}

int dp_allreduce_sum_f32(DpState* d, float* buf, long long n, cudaStream_t s) {
  if (!d) return 0;
  if (!d->comm) return femto_fail(FEMTO_ERR_STATE, "the communicator was aborted");
  return nccl_check(g_nccl.allreduce(buf, buf, (size_t)n, NCCL_FLOAT32, NCCL_SUM, d->comm, s), "ncclAllReduce");
}
int dp_allreduce_sum_bf16(DpState* d, void* buf, long long n, cudaStream_t s) {
  if (!d) return 0;
  if (!d->comm) return femto_fail(FEMTO_ERR_STATE, "the communicator was aborted");
  return nccl_check(g_nccl.allreduce(buf, buf, (size_t)n, NCCL_BFLOAT16, NCCL_SUM, d->comm, s), "ncclAllReduce");
}
int dp_allreduce_sum_i32(DpState* d, int* buf, long long n, cudaStream_t s) {
  if (!d) return 0;
  if (!d->comm) return femto_fail(FEMTO_ERR_STATE, "the communicator was aborted");
  return nccl_check(g_nccl.allreduce(buf, buf, (size_t)n, NCCL_INT32, NCCL_SUM, d->comm, s), "ncclAllReduce");
}
// Gradient sum for the owner-sharded update: every range of delta is summed over ranks, but a range that one rank alone
// will consume is summed only onto that rank (in-place reduce-scatter of the sliced tables, reduce to the owner of
// each (offset, count, owner) run), which moves half the bytes of an all-reduce; `gaps` (offset, count) are the
// replicated ranges in between and get a plain all-reduce.  One NCCL group on `s`.
int dp_reduce_ranges(DpState* d, float* delta, const long long* gathers, int n_gathers, const long long* bcasts,
                     int n_bcasts, const long long* gaps, int n_gaps, cudaStream_t s) {
  if (!d) return 0;
  if (!d->comm) return femto_fail(FEMTO_ERR_STATE, "the communicator was aborted");
  FEMTO_TRY(nccl_check(g_nccl.group_start(), "ncclGroupStart"));
  int r = 0;
  for (int i = 0; i < n_gathers && !r; i++) {
    float* base = delta + gathers[2 * i];
    const long long c = gathers[2 * i + 1];
    r = g_nccl.reduce_scatter(base, base + (long long)d->rank * c, (size_t)c, NCCL_FLOAT32, NCCL_SUM, d->comm, s);
  }
  for (int i = 0; i < n_bcasts && !r; i++) {
    float* p = delta + bcasts[3 * i];
    r = g_nccl.reduce(p, p, (size_t)bcasts[3 * i + 1], NCCL_FLOAT32, NCCL_SUM, (int)bcasts[3 * i + 2], d->comm, s);
  }
  for (int i = 0; i < n_gaps && !r; i++) {
    float* p = delta + gaps[2 * i];
    r = g_nccl.allreduce(p, p, (size_t)gaps[2 * i + 1], NCCL_FLOAT32, NCCL_SUM, d->comm, s);
  }
  const int e = g_nccl.group_end();
  FEMTO_TRY(nccl_check(r, "ncclReduceScatter / ncclReduce / ncclAllReduce"));
  return nccl_check(e, "ncclGroupEnd");
}
// Asynchronous errors of the communicator (a peer that died, a network fault): collectives are only checked when they
// are enqueued, so a host loop polls this between steps.  0 = healthy or still in progress (ncclInProgress = 7).
int dp_async_error(DpState* d) {
  if (!d || !d->comm || !g_nccl.async_err) return 0;
  int state = 0;
  const int r = g_nccl.async_err(d->comm, &state);
  if (r != 0) return nccl_check(r, "ncclCommGetAsyncError");
  if (state == 0 || state == 7) return 0;
  return nccl_check(state, "NCCL communicator (asynchronous error)");
}
// Tear the communicator down without waiting for outstanding collectives (after dp_async_error reported a fault or a
// host-side timeout expired): afterwards the handle has no communicator and data-parallel calls fail cleanly.
int dp_abort(DpState* d) {
  if (!d || !d->comm) return 0;
  int r = 0;
  if (g_nccl.abort) r = g_nccl.abort(d->comm);
  d->comm = nullptr;
  return nccl_check(r, "ncclCommAbort");
}
bool dp_alive(const DpState* d) { return d && d->comm; }
int dp_world(const DpState* d) { return d ? d->world : 1; }
int dp_rank(const DpState* d) { return d ? d->rank : 0; }
