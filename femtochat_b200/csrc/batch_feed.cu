// Packed-batch producer on the device and a pinned, double-buffered host feeder: the step either side of the
// gradient driver (src/dataloader.jl:241-274 `model_batch!`, and the host-to-device copy of every micro-step,
// scripts/train.jl:144-145).
//
// model_batch! copies runs of documents into B columns of T rows: tokens, targets (the next token of the
// stream; a document's last token predicts BOS) and positions (restarting at 0 on BOS).  Which document goes
// to which column depends only on the document lengths, so the host keeps that O(#documents) bookkeeping and
// hands the device a list of segments; the O(tokens) work (widening 16-bit token ids, shifting targets,
// counting positions) is an HBM-streaming kernel over the token stream as it lies in device memory.
#include <string.h>

#include <vector>

#include "common.cuh"

namespace {

// rows not covered by a segment are padding: token = BOS, target = -1, position = 0 (src/dataloader.jl:243-245)
__global__ void __launch_bounds__(256) k_pack_fill(int* __restrict__ tokens, int* __restrict__ targets,
                                                   int* __restrict__ positions, long long n, int bos) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  tokens[i] = bos;
  targets[i] = -1;
  positions[i] = 0;
}

// One block per (segment, 2048-row chunk).  Row i of a segment: token = stream[src + i], position = pos0 + i,
// target = stream[src + i + 1], except the last row whose target is the segment's `next` (the next token of the
// document when it continues in the next batch, BOS when it ends there).
__global__ void __launch_bounds__(256) k_pack_segments(const uint16_t* __restrict__ stream0, long long n_stream,
                                                       const femto_segment* __restrict__ segs, int B, int T, int base,
                                                       int* __restrict__ tokens, int* __restrict__ targets,
                                                       int* __restrict__ positions, unsigned int* status) {
  const femto_segment sg = segs[blockIdx.x];
  const int i0 = blockIdx.y * 2048;
  if (i0 >= sg.n) return;
  const bool bad = sg.col < 0 || sg.col >= B || sg.row < 0 || sg.n < 0 || sg.row + sg.n > T || sg.src < 0 ||
                   sg.src + sg.n > n_stream;
  if (bad) {   // a segment outside the batch or the stream is skipped and flagged, never dereferenced
    if (threadIdx.x == 0 && status) atomicOr(status, ST_BAD_TOKEN);
    return;
  }
  const long long out0 = (long long)sg.col * T + sg.row;
  const int i1 = min(sg.n, i0 + 2048);
  for (int i = i0 + threadIdx.x; i < i1; i += 256) {
    const int tk = stream0[sg.src + i];
    int tg;
    if (i + 1 < sg.n) tg = (int)stream0[sg.src + i + 1] + base;
    else tg = sg.next < 0 ? -1 : sg.next + base;
    tokens[out0 + i] = tk + base;
    targets[out0 + i] = tg;
    positions[out0 + i] = sg.pos0 + i;
  }
}

}  // namespace

extern "C" int32_t femto_pack_batch(const uint16_t* stream0, int64_t n_stream, const femto_segment* segments,
                                    int32_t n_segments, int32_t B, int32_t T, int32_t bos0, int32_t index_base,
                                    int32_t* tokens, int32_t* targets, int32_t* positions, uint32_t* status,
                                    void* stream) {
  if (!stream0 || !tokens || !targets || !positions || (n_segments > 0 && !segments) || B <= 0 || T <= 0 ||
      n_segments < 0 || n_stream < 0)
    return femto_fail(FEMTO_ERR_ARG, "bad argument");
  if (index_base != 0 && index_base != 1) return femto_fail(FEMTO_ERR_ARG, "index_base must be 0 or 1");
  cudaStream_t s = (cudaStream_t)stream;
  const long long n = (long long)B * T;
  k_pack_fill<<<cdiv(n, 256), 256, 0, s>>>(tokens, targets, positions, n, bos0 + index_base);
  KERNEL_CHECK();
  if (n_segments > 0) {
    k_pack_segments<<<dim3(n_segments, cdiv(T, 2048)), 256, 0, s>>>(stream0, n_stream, segments, B, T, index_base, tokens,
                                                                    targets, positions, status);
    KERNEL_CHECK();
  }
  return 0;
}

// ---- feeder --------------------------------------------------------------------------------------------------
// `depth` slots, each a pinned host staging area and a device area for the three int32 [B][T] arrays, one copy
// stream and one event per slot.  submit() copies the caller's arrays into the slot's pinned area and queues the
// host-to-device copy on the copy stream; next() makes the compute stream wait for that copy and hands out the
// device pointers.  While the GPU works on batch i the host is free to submit batch i+1.
struct femto_feeder {
  int B = 0, T = 0, depth = 0;
  size_t bytes = 0;                // of one array
  std::vector<int*> host, dev;     // [depth] bases; arrays at +0, +n, +2n
  std::vector<cudaEvent_t> copied, consumed;
  std::vector<char> has_pos, pending_consume, used;
  bool last_released = true;       // the batch handed out by the last next() has been released
  cudaStream_t copy = nullptr;
  long long submitted = 0, taken = 0;
};

extern "C" int32_t femto_feeder_create(int32_t B, int32_t T, int32_t depth, femto_feeder** out) {
  if (!out || B <= 0 || T <= 0 || depth < 1 || depth > 16) return femto_fail(FEMTO_ERR_ARG, "bad argument");
  *out = nullptr;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
    return femto_fail(FEMTO_ERR_UNSUPPORTED, "no CUDA device: libfemto_sm100a has no CPU fallback");
  femto_feeder* f = new femto_feeder();
  f->B = B; f->T = T; f->depth = depth;
  f->bytes = sizeof(int) * (size_t)B * T;
  f->host.assign(depth, nullptr); f->dev.assign(depth, nullptr);
  f->copied.assign(depth, nullptr); f->consumed.assign(depth, nullptr);
  f->has_pos.assign(depth, 0); f->pending_consume.assign(depth, 0); f->used.assign(depth, 0);
  auto fail = [&](cudaError_t e, const char* what) {
    int rc = femto_fail(e == cudaErrorMemoryAllocation ? FEMTO_ERR_NOMEM : (int)e, "%s failed: %s", what, cudaGetErrorString(e));
    for (int i = 0; i < depth; i++) {
      if (f->host[i]) cudaFreeHost(f->host[i]);
      if (f->dev[i]) cudaFree(f->dev[i]);
      if (f->copied[i]) cudaEventDestroy(f->copied[i]);
      if (f->consumed[i]) cudaEventDestroy(f->consumed[i]);
    }
    if (f->copy) cudaStreamDestroy(f->copy);
    delete f;
    return rc;
  };
  cudaError_t e = cudaStreamCreateWithFlags(&f->copy, cudaStreamNonBlocking);
  if (e != cudaSuccess) return fail(e, "cudaStreamCreate");
  for (int i = 0; i < depth; i++) {
    if ((e = cudaMallocHost(&f->host[i], 3 * f->bytes)) != cudaSuccess) return fail(e, "cudaMallocHost");
    if ((e = cudaMalloc(&f->dev[i], 3 * f->bytes)) != cudaSuccess) return fail(e, "cudaMalloc");
    if ((e = cudaEventCreateWithFlags(&f->copied[i], cudaEventDisableTiming)) != cudaSuccess) return fail(e, "cudaEventCreate");
    if ((e = cudaEventCreateWithFlags(&f->consumed[i], cudaEventDisableTiming)) != cudaSuccess) return fail(e, "cudaEventCreate");
  }
  *out = f;
  return 0;
}

extern "C" int32_t femto_feeder_destroy(femto_feeder* f) {
  if (!f) return 0;
  cudaStreamSynchronize(f->copy);
  for (int i = 0; i < f->depth; i++) {
    cudaFreeHost(f->host[i]); cudaFree(f->dev[i]);
    cudaEventDestroy(f->copied[i]); cudaEventDestroy(f->consumed[i]);
  }
  cudaStreamDestroy(f->copy);
  delete f;
  return 0;
}

extern "C" int32_t femto_feeder_submit(femto_feeder* f, const int32_t* h_tokens, const int32_t* h_targets,
                                       const int32_t* h_positions) {
  if (!f || !h_tokens || !h_targets) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  if (f->submitted - f->taken >= f->depth)
    return femto_fail(FEMTO_ERR_STATE, "feeder is full: %d batches submitted and not yet taken", f->depth);
  const int slot = (int)(f->submitted % f->depth);
  // The pinned area is read only by the slot's previous host-to-device copy: the host waits for that copy (short).
  // The device area may still be read by the step that took the previous batch: the COPY STREAM waits for that
  // step, the host does not.
  if (f->used[slot]) CUDA_TRY(cudaEventSynchronize(f->copied[slot]));
  if (f->pending_consume[slot]) {
    CUDA_TRY(cudaStreamWaitEvent(f->copy, f->consumed[slot], 0));
    f->pending_consume[slot] = 0;
  }
  f->used[slot] = 1;
  const size_t n = (size_t)f->B * f->T;
  memcpy(f->host[slot], h_tokens, f->bytes);
  memcpy(f->host[slot] + n, h_targets, f->bytes);
  f->has_pos[slot] = h_positions != nullptr;
  if (h_positions) memcpy(f->host[slot] + 2 * n, h_positions, f->bytes);
  CUDA_TRY(cudaMemcpyAsync(f->dev[slot], f->host[slot], (h_positions ? 3 : 2) * f->bytes, cudaMemcpyHostToDevice, f->copy));
  CUDA_TRY(cudaEventRecord(f->copied[slot], f->copy));
  f->submitted++;
  return 0;
}

extern "C" int32_t femto_feeder_release(femto_feeder* f, void* compute_stream);

extern "C" int32_t femto_feeder_next(femto_feeder* f, void* compute_stream, const int32_t** d_tokens,
                                     const int32_t** d_targets, const int32_t** d_positions) {
  if (!f || !d_tokens || !d_targets || !d_positions) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  if (f->taken >= f->submitted) return femto_fail(FEMTO_ERR_STATE, "feeder is empty: submit a batch first");
  const int slot = (int)(f->taken % f->depth);
  cudaStream_t s = (cudaStream_t)compute_stream;
  // a batch that was never released explicitly counts as consumed by whatever is on the compute stream by now
  if (!f->last_released) FEMTO_TRY(femto_feeder_release(f, compute_stream));
  f->last_released = false;
  CUDA_TRY(cudaStreamWaitEvent(s, f->copied[slot], 0));
  const size_t n = (size_t)f->B * f->T;
  *d_tokens = f->dev[slot];
  *d_targets = f->dev[slot] + n;
  *d_positions = f->has_pos[slot] ? f->dev[slot] + 2 * n : nullptr;
  f->taken++;
  return 0;
}

// Call after the work that reads the batch handed out by the last femto_feeder_next has been queued on the compute
// stream: marks the point after which that slot may be refilled.
extern "C" int32_t femto_feeder_release(femto_feeder* f, void* compute_stream) {
  if (!f) return femto_fail(FEMTO_ERR_ARG, "NULL argument");
  if (f->taken == 0) return femto_fail(FEMTO_ERR_STATE, "nothing taken yet");
  const int slot = (int)((f->taken - 1) % f->depth);
  CUDA_TRY(cudaEventRecord(f->consumed[slot], (cudaStream_t)compute_stream));
  f->pending_consume[slot] = 1;
  f->last_released = true;
  return 0;
}
