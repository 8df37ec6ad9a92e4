// Deterministic segmented embedding-gradient scatter: table[tok[n]] += dy[n]
// (reference: sequential CPU loop src/kernels.jl:8-14; its GPU form uses fp32 atomics,
// ext/FemtoChatCUDAExt.jl:77-94, whose rounding depends on arrival order).
//
// The token list is sorted once per batch (stable radix sort, so occurrences of a token stay in
// token order), run-length encoded into segments, and each segment is cut into chunks of CH
// occurrences.  One block sums one chunk in order; a segment with one chunk adds straight into
// the table, longer segments (BOS, the head of the Zipf distribution) go through per-chunk
// partial rows that a second kernel adds up in chunk order.  The plan is shared by the token
// embedding and every value-embedding table of the step.
#include <cub/cub.cuh>

#include "common.cuh"

constexpr int CH = 32;

struct ScatterPlan {
  int N = 0, max_cols = 0, cur = 0;  // capacity, widest row, tokens of the current batch
  int *iota = nullptr, *sorted_tok = nullptr, *order = nullptr, *uniq = nullptr, *counts = nullptr, *num_runs = nullptr;
  int *seg_start = nullptr, *nchunks = nullptr, *chunk_start = nullptr, *pchunks = nullptr, *pstart = nullptr;
  float* partial = nullptr;
  void* tmp = nullptr;
  size_t tmp_bytes = 0;
  int max_partial_rows = 0;
  int bits = 32;
};

namespace {

__global__ void k_iota(int* p, int n) {
  pdl_trigger();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = i;
}
__global__ void k_chunks(const int* counts, const int* num_runs, int n, int* nchunks, int* pchunks) {
  pdl_trigger();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int c = i < num_runs[0] ? counts[i] : 0;
  int nc = (c + CH - 1) / CH;
  nchunks[i] = nc;
  pchunks[i] = nc > 1 ? nc : 0;
}

// One WARP per chunk (eight chunks per block): a chunk is at most CH rows of D columns, far too little for a block, and
// with one block per possible chunk two thirds of the blocks found nothing to do.  The lanes cover the columns with
// 16-byte loads; the chunk's row indices are read once (lane r holds row r) and passed round by shuffle.
template <typename T, int V>
__global__ void __launch_bounds__(256) k_scatter_chunks(const int* __restrict__ num_runs, const int* __restrict__ uniq,
                                                        const int* __restrict__ counts,
                                                        const int* __restrict__ seg_start,
                                                        const int* __restrict__ chunk_start,
                                                        const int* __restrict__ nchunks,
                                                        const int* __restrict__ pstart, const int* __restrict__ order,
                                                        const T* __restrict__ dy, long long dy_stride, int D,
                                                        float* __restrict__ table, float* __restrict__ partial, int n) {
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int nr = num_runs[0];
  const int total = chunk_start[nr - 1] + nchunks[nr - 1];
  const int item = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (item >= total) return;
  // binary search: last segment with chunk_start <= item
  int lo = 0, hi = nr - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (chunk_start[mid] <= item) lo = mid; else hi = mid - 1;
  }
  const int seg = lo;
  const int ck = item - chunk_start[seg];
  const int first = seg_start[seg] + ck * CH;
  const int cnt = min(CH, counts[seg] - ck * CH);
  const bool direct = nchunks[seg] == 1;
  float* dst = direct ? table + (long long)uniq[seg] * D : partial + (long long)(pstart[seg] + ck) * D;
  static_assert(CH <= 32, "a lane holds one row index of the chunk");
  const int my_row = lane < cnt ? order[first + lane] : 0;
  for (int c0 = 0; c0 < D; c0 += 32 * V) {   // every lane walks every pass: the shuffles below need the whole warp
    const int c = c0 + lane * V;
    const bool live = c < D;
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; i++) acc[i] = 0.f;
    for (int r = 0; r < cnt; r++) {   // in token order: the sum is repeatable
      const int row = __shfl_sync(0xffffffffu, my_row, r);
      if (live) {
        float f[V];
        load_vec<T, V>(dy + (long long)row * dy_stride + c, f);
#pragma unroll
        for (int i = 0; i < V; i++) acc[i] += f[i];
      }
    }
    if (live) {
#pragma unroll
      for (int i = 0; i < V; i++) dst[c + i] = direct ? dst[c + i] + acc[i] : acc[i];
    }
  }
}

// Segments with more than one chunk (BOS, the head of the token distribution): their partial rows are added up in
// chunk order.  A block looks at 256 segments at once and handles the few that qualify one after the other.
__global__ void __launch_bounds__(256) k_scatter_combine(const int* __restrict__ num_runs, const int* __restrict__ uniq,
                                                         const int* __restrict__ nchunks,
                                                         const int* __restrict__ pstart, int D,
                                                         float* __restrict__ table, const float* __restrict__ partial) {
  pdl_trigger();
  __shared__ int s_list[256];
  __shared__ int s_cnt;
  const int nr = num_runs[0];
  // thread t of block b looks at segment t * gridDim.x + b (+ whole rounds): neighbouring segments, and the frequent
  // tokens are neighbours, go to different blocks
  for (int base = 0; base < nr; base += gridDim.x * 256) {
    if (threadIdx.x == 0) s_cnt = 0;
    __syncthreads();
    const int mine = base + threadIdx.x * gridDim.x + blockIdx.x;
    if (mine < nr && nchunks[mine] > 1) s_list[atomicAdd(&s_cnt, 1)] = mine;   // the order of the list does not matter:
    __syncthreads();                                                           // every segment has its own row
    const int cnt = s_cnt;
    for (int k = 0; k < cnt; k++) {
      const int seg = s_list[k];
      const int nc = nchunks[seg];
      float* dst = table + (long long)uniq[seg] * D;
      const float* src = partial + (long long)pstart[seg] * D;
      if ((D & 3) == 0) {
        // four columns per thread and sixteen chunks in flight, added in chunk order: the head of the token
        // distribution has hundreds of chunks, and one dependent load per chunk bounded the whole kernel
        for (int c = threadIdx.x * 4; c < D; c += 1024) {
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
          int j = 0;
          for (; j + 16 <= nc; j += 16) {
            float4 v[16];
#pragma unroll
            for (int u = 0; u < 16; u++) v[u] = *reinterpret_cast<const float4*>(src + (long long)(j + u) * D + c);
#pragma unroll
            for (int u = 0; u < 16; u++) { acc[0] += v[u].x; acc[1] += v[u].y; acc[2] += v[u].z; acc[3] += v[u].w; }
          }
          for (; j < nc; j++) {
            const float4 v = *reinterpret_cast<const float4*>(src + (long long)j * D + c);
            acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
          }
#pragma unroll
          for (int i = 0; i < 4; i++) dst[c + i] += acc[i];
        }
      } else {
        for (int c = threadIdx.x; c < D; c += 256) {
          float acc = 0.f;
          for (int j = 0; j < nc; j++) acc += src[(long long)j * D + c];
          dst[c] += acc;
        }
      }
    }
    __syncthreads();
  }
}

}  // namespace

int scatter_plan_create(ScatterPlan** out, int N, int max_cols) {
  ScatterPlan* p = new ScatterPlan();
  p->N = N;
  p->max_cols = max_cols;
  p->max_partial_rows = 2 * (N / CH) + 4;
  size_t t1 = 0, t2 = 0, t3 = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, t1, (int*)nullptr, (int*)nullptr, (int*)nullptr, (int*)nullptr, N);
  cub::DeviceRunLengthEncode::Encode(nullptr, t2, (int*)nullptr, (int*)nullptr, (int*)nullptr, (int*)nullptr, N);
  cub::DeviceScan::ExclusiveSum(nullptr, t3, (int*)nullptr, (int*)nullptr, N);
  p->tmp_bytes = std::max(t1, std::max(t2, t3)) + 256;
  int** arrs[] = {&p->iota, &p->sorted_tok, &p->order, &p->uniq, &p->counts, &p->seg_start,
                  &p->nchunks, &p->chunk_start, &p->pchunks, &p->pstart};
  for (auto a : arrs) {
    CUDA_TRY(cudaMalloc(a, sizeof(int) * (size_t)(N + 1)));
    CUDA_TRY(cudaMemset(*a, 0, sizeof(int) * (size_t)(N + 1)));
  }
  CUDA_TRY(cudaMalloc(&p->num_runs, sizeof(int)));
  CUDA_TRY(cudaMalloc(&p->partial, sizeof(float) * (size_t)p->max_partial_rows * max_cols));
  CUDA_TRY(cudaMalloc(&p->tmp, p->tmp_bytes));
  *out = p;
  return 0;
}

void scatter_plan_destroy(ScatterPlan* p) {
  if (!p) return;
  int* arrs[] = {p->iota, p->sorted_tok, p->order, p->uniq, p->counts, p->seg_start,
                 p->nchunks, p->chunk_start, p->pchunks, p->pstart, p->num_runs};
  for (auto a : arrs) cudaFree(a);
  cudaFree(p->partial);
  cudaFree(p->tmp);
  delete p;
}

int scatter_plan_build(ScatterPlan* p, const int* tokens0, int N, int rows, cudaStream_t s) {
  if (N > p->N) return femto_fail(FEMTO_ERR_SHAPE, "scatter plan built for %d tokens, got %d", p->N, N);
  p->cur = N;
  int bits = 1;
  while ((1ll << bits) < rows) bits++;
  k_iota<<<cdiv(N, 256), 256, 0, s>>>(p->iota, N);
  KERNEL_CHECK();
  size_t tb = p->tmp_bytes;
  CUDA_TRY(cub::DeviceRadixSort::SortPairs(p->tmp, tb, tokens0, p->sorted_tok, p->iota, p->order, N, 0, bits, s));
  LAUNCH_COUNT();
  tb = p->tmp_bytes;
  CUDA_TRY(cub::DeviceRunLengthEncode::Encode(p->tmp, tb, p->sorted_tok, p->uniq, p->counts, p->num_runs, N, s));
  LAUNCH_COUNT();
  k_chunks<<<cdiv(N, 256), 256, 0, s>>>(p->counts, p->num_runs, N, p->nchunks, p->pchunks);
  KERNEL_CHECK();
  // counts beyond num_runs are stale: scan the masked copy instead (nchunks==0 there), and build
  // seg_start from a masked count array held in pstart temporarily.
  tb = p->tmp_bytes;
  CUDA_TRY(cub::DeviceScan::ExclusiveSum(p->tmp, tb, p->nchunks, p->chunk_start, N, s));
  tb = p->tmp_bytes;
  CUDA_TRY(cub::DeviceScan::ExclusiveSum(p->tmp, tb, p->pchunks, p->pstart, N, s));
  tb = p->tmp_bytes;
  CUDA_TRY(cub::DeviceScan::ExclusiveSum(p->tmp, tb, p->counts, p->seg_start, N, s));
  g_femto_launches += 3;
  return 0;
}

template <typename T>
int scatter_rows(ScatterPlan* p, float* table, const T* dy, long long dy_stride, int D, cudaStream_t s) {
  if (D > p->max_cols) return femto_fail(FEMTO_ERR_SHAPE, "scatter: D=%d exceeds plan width %d", D, p->max_cols);
  const int N = p->cur;
  const int grid = cdiv(N / CH + N + 1, 8);  // eight chunks per block; the count is an upper bound, surplus warps exit at once
  const bool vec = D % VecN<T>::n == 0 && dy_stride % VecN<T>::n == 0 && aligned16(dy);
  if (vec)
    k_scatter_chunks<T, VecN<T>::n><<<grid, 256, 0, s>>>(p->num_runs, p->uniq, p->counts, p->seg_start, p->chunk_start,
                                                       p->nchunks, p->pstart, p->order, dy, dy_stride, D, table,
                                                       p->partial, N);
  else
    k_scatter_chunks<T, 1><<<grid, 256, 0, s>>>(p->num_runs, p->uniq, p->counts, p->seg_start, p->chunk_start,
                                              p->nchunks, p->pstart, p->order, dy, dy_stride, D, table, p->partial, N);
  KERNEL_CHECK();
  k_scatter_combine<<<std::min(cdiv(N, 256), 1184), 256, 0, s>>>(p->num_runs, p->uniq, p->nchunks, p->pstart, D, table, p->partial);
  KERNEL_CHECK();
  return 0;
}
template int scatter_rows<float>(ScatterPlan*, float*, const float*, long long, int, cudaStream_t);
template int scatter_rows<bf16>(ScatterPlan*, float*, const bf16*, long long, int, cudaStream_t);
