// Flash attention for head_dim 128 in bf16 on the sm_100a tensor cores: causal mask with a
// sliding window (keys t-left..t) and an optional per-document lower bound, GQA by
// kv_head = head / (H/Hkv).  Replaces the reference's mma.sync kernels
// (ext/FemtoChatCUDAExt.jl:1295-1463 forward, :1829-2068 reverse); arithmetic follows
// src/kernels.jl:131-219 and :287-379 (softmax in base 2, fp32 statistics).
//
// Forward: one CTA owns 128 queries of one (batch, head).  Warp 0 streams K/V tiles of 128 keys
// with TMA (two stages each).  Warp 1 issues S = Q K^T into one of two 128-column TMEM buffers and
// warp 2 issues O += P V with P read back from TMEM (P overwrites S in place as bf16): tcgen05.mma
// issue blocks while the pipe is busy, so with one issuer per product the barrier waits of one
// overlap the issue of the other.  Warps 4-11 own the query rows, two threads per row (64 keys
// each): they read S with tcgen05.ld, keep the running max / sum, rescale the TMEM-resident O only
// when the max grew by more than 2^8, and write P with tcgen05.st.  S of tile j+1 is computed
// while the softmax of tile j runs.
#include <stdio.h>
#include <stdlib.h>

#include <algorithm>

#include "sm100_ptx.cuh"

using namespace sm100;

namespace {

constexpr int HD = 128, BQ = 128, BKV = 128;
constexpr int NS = 2;              // threads per query row in the forward softmax (4 measured slower: 583 vs 620 TFLOP/s)
constexpr int CW = BKV / NS;       // keys of a tile per thread
constexpr int FWD_THREADS = 128 + NS * 128;
constexpr int TILE_BYTES = BQ * HD * 2;  // 32 KB: two [128][64] swizzled slabs
constexpr int FWD_SMEM = TILE_BYTES * 5 + 1024 + 256 + 3 * NS * 128 * 4;
constexpr float LOG2E = 1.4426950408889634f;

struct FwdParams {
  AttnArgs a;
  int q_col0, k_col0, v_col0;  // column offsets (elements) of head 0 inside the Q / K / V tensor maps
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Optional cycle accounting of the roles of the persistent forward kernels (compiled in with -DFEMTO_ATTN_CYCLES,
// printed by the launcher when FEMTO_ATTN_PROF is set in the environment): consecutive laps of clock64(), summed per
// role in CTA 0.  In a normal build every member is empty.
struct Cyc {
#ifdef FEMTO_ATTN_CYCLES
  long long t = 0, acc[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
  __device__ __forceinline__ void start() { t = clock64(); }
  __device__ __forceinline__ void lap(int i) { const long long n = clock64(); acc[i] += n - t; t = n; }
  __device__ __forceinline__ void store(long long* prof, int slot, int tiles) const {
    if (!prof || blockIdx.x != 0) return;
    for (int i = 0; i < 10; i++) prof[slot * 16 + i] = acc[i];
    prof[slot * 16 + 10] = tiles;
  }
#else
  __device__ __forceinline__ void start() {}
  __device__ __forceinline__ void lap(int) {}
  __device__ __forceinline__ void store(long long*, int, int) const {}
#endif
};

__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const FwdParams p) {
  grid_launch_dependents();   // the GEMM that follows may set itself up while this kernel runs (it still waits for our completion)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + TILE_BYTES;       // 2 stages
  uint8_t* sV = smem + 3 * TILE_BYTES;   // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 5 * TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* v_full = bars + 3;    // [2]
  uint64_t* s_full = bars + 5;    // [2] S of a tile is in TMEM; also frees the tile's K stage
  uint64_t* p_ready = bars + 7;   // [2]
  uint64_t* pv_done = bars + 9;   // [2] P V of a tile has been accumulated; also frees its V stage and its S/P buffer
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xmax = reinterpret_cast<float*>(smem + 5 * TILE_BYTES + 256);  // [2 parities][NS][128 rows]
  float* xl = xmax + 2 * NS * 128;                                      // [NS][128 rows]

  const AttnArgs& a = p.a;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;  // heavy (late) query tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (a.H / a.Hkv);
  const int q0 = qt * BQ;
  const int jhi = min(q0 + BQ - 1, a.T - 1) / BKV;
  int jlo = max(0, q0 - a.window_left) / BKV;
  const long long row0 = (long long)b * a.T;
  if (a.doc_start) {
    // key tiles that lie before the earliest document start of these 128 queries are fully masked
    __shared__ int s_ds_min[4];
    if (threadIdx.x < 128) {
      const int qq = min(q0 + (int)threadIdx.x, a.T - 1);
      const int v = __reduce_min_sync(0xffffffffu, a.doc_start[row0 + qq]);
      if ((threadIdx.x & 31) == 0) s_ds_min[threadIdx.x >> 5] = v;
    }
    __syncthreads();
    jlo = max(jlo, min(min(s_ds_min[0], s_ds_min[1]), min(s_ds_min[2], s_ds_min[3])) / BKV);
  }
  const int ntile = jhi - jlo + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; i++) {
      mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_ready[i], NS * 4); mbar_init(&pv_done[i], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS[2] = {tmem_base, tmem_base + 128};
  const uint32_t tO = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer ----------------
      mbar_expect_tx(q_full, TILE_BYTES);
      tma_load_2d(sQ, &tmQ, q_full, p.q_col0 + h * HD, (int)(row0 + q0));
      tma_load_2d(sQ + TILE_BYTES / 2, &tmQ, q_full, p.q_col0 + h * HD + 64, (int)(row0 + q0));
      bool ok = true;
      for (int i = 0; i < ntile && ok; i++) {
        const int st = i & 1;
        const uint32_t ph2 = ((i - 2) >> 1) & 1;   // phase of tile i-2, the previous user of this stage
        const int krow = (int)(row0 + (jlo + i) * BKV);
        if (i >= 2 && !mbar_wait(&s_full[st], ph2, abort_flag, a.status)) { ok = false; break; }
        mbar_expect_tx(&k_full[st], TILE_BYTES);
        tma_load_2d(sK + st * TILE_BYTES, &tmK, &k_full[st], p.k_col0 + kvh * HD, krow);
        tma_load_2d(sK + st * TILE_BYTES + TILE_BYTES / 2, &tmK, &k_full[st], p.k_col0 + kvh * HD + 64, krow);
        if (i >= 2 && !mbar_wait(&pv_done[st], ph2, abort_flag, a.status)) { ok = false; break; }
        mbar_expect_tx(&v_full[st], TILE_BYTES);
        tma_load_2d(sV + st * TILE_BYTES, &tmV, &v_full[st], p.v_col0 + kvh * HD, krow);
        tma_load_2d(sV + st * TILE_BYTES + TILE_BYTES / 2, &tmV, &v_full[st], p.v_col0 + kvh * HD + 64, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- S = Q K^T issuer ----------------
      // The two products of a tile are issued by different threads, so the barrier waits of one overlap
      // the (blocking) instruction issue of the other and the tensor pipe is fed from whichever is ready.
      constexpr uint32_t idesc_s = idesc_bf16(BQ, BKV, false, false);  // both operands K-major
      const uint32_t q_addr = smem_u32(sQ);
      bool ok = mbar_wait(q_full, 0, abort_flag, a.status);
      for (int i = 0; i < ntile && ok; i++) {
        const int st = i & 1;
        if (!mbar_wait(&k_full[st], (i >> 1) & 1, abort_flag, a.status)) break;
        // S(i) overwrites the buffer that held P(i-2): its P V must have been executed
        if (i >= 2 && !mbar_wait(&pv_done[st], ((i - 2) >> 1) & 1, abort_flag, a.status)) break;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + st * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; k++) {
          const uint32_t off = (k >> 2) * (TILE_BYTES / 2) + (k & 3) * 32;
          mma_ss(tS[st], smem_desc_sw128(q_addr + off, 16, 1024), smem_desc_sw128(k_addr + off, 16, 1024), idesc_s, k > 0);
        }
        tc_commit(&s_full[st]);
      }
    }
  } else if (warp == 2) {
    if (lane == 0) {
      // ---------------- O += P V issuer ----------------
      constexpr uint32_t idesc_o = idesc_bf16(BQ, HD, false, true);    // V is N-contiguous
      for (int i = 0; i < ntile; i++) {
        const int st = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(&p_ready[st], ph, abort_flag, a.status)) break;
        if (!mbar_wait(&v_full[st], ph, abort_flag, a.status)) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + st * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < BKV / 16; k++) {
          // A: 16 keys of P = 8 TMEM columns; B: 16 key rows of the [128][64] slabs = 2048 B, the two
          // 64-wide head_dim halves 16 KB apart.
          mma_ts(tO, tS[st] + k * 8, smem_desc_sw128(v_addr + k * 2048, TILE_BYTES / 2, 1024), idesc_o, (i > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(&pv_done[st]);
      }
    }
  } else if (warp >= 4) {
    // ---------------- softmax: NS threads per query row, each owns CW = 128 / NS of the keys of a tile ----------------
    const int quad = warp & 3;
    const int hs = (warp - 4) >> 2;        // which CW keys of each tile
    const int r = quad * 32 + lane;
    const int q = q0 + r;
    const bool row_ok = q < a.T;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const float c = rsqrtf((float)HD) * LOG2E;
    int lo = max(0, q - a.window_left);
    if (a.doc_start && row_ok) lo = max(lo, a.doc_start[row0 + q]);
    float m_used = -INFINITY, l = 0.f;   // l: this thread's share of the row sum (same m_used in all threads of a row)
    bool ok = true;
    for (int i = 0; i < ntile; i++) {
      const int st = i & 1;
      const uint32_t ph = (i >> 1) & 1;
      const int k0 = (jlo + i) * BKV + hs * CW;
      // After a timed-out wait the warp keeps walking the loop (skipping the work) so that it still
      // meets its partner warps at every row barrier.
      if (ok && !mbar_wait(&s_full[st], ph, abort_flag, a.status)) ok = false;
      if (!ok) { asm volatile("bar.sync %0, %1;" ::"r"(2 + quad), "n"(NS * 32) : "memory"); continue; }
      tc_fence_after();
      // x holds the raw scores; the 1/sqrt(hd) * log2(e) factor is folded into the exponent's FMA.
      // Maxima and sums use four independent accumulators so the chains do not serialise.
      float x[CW];
#pragma unroll
      for (int u = 0; u < CW / 32; u++)
        tmem_ld32(tS[st] + lane_off + hs * CW + u * 32, *reinterpret_cast<uint32_t(*)[32]>(&x[u * 32]));
      tmem_ld_wait();
      const bool need_mask = (k0 + CW - 1 > q) || (k0 < lo);
      if (need_mask) {
#pragma unroll
        for (int j = 0; j < CW; j++) {
          const int k = k0 + j;
          x[j] = (k <= q && k >= lo) ? x[j] : -INFINITY;
        }
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < CW; j += 4) {
        mx[0] = fmaxf(mx[0], x[j]); mx[1] = fmaxf(mx[1], x[j + 1]);
        mx[2] = fmaxf(mx[2], x[j + 2]); mx[3] = fmaxf(mx[3], x[j + 3]);
      }
      float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * c;   // scaled units (c > 0 keeps the argmax)
      // combine the partial row maxima; after this barrier every thread of the row holds its part of S in
      // registers, so P may overwrite S in TMEM
      xmax[(i & 1) * (NS * 128) + hs * 128 + r] = mt;
      asm volatile("bar.sync %0, %1;" ::"r"(2 + quad), "n"(NS * 32) : "memory");
#pragma unroll
      for (int o = 1; o < NS; o++) mt = fmaxf(mt, xmax[(i & 1) * (NS * 128) + ((hs + o) % NS) * 128 + r]);
      const bool grow = mt > m_used + 8.f || (m_used == -INFINITY && mt > -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_used, mt);
        const float alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new);
        l *= alpha;
        m_used = m_new;
        if (i > 0) {
          // O lives in TMEM and is being accumulated by the tensor core: wait for tile i-1's P V
          if (!mbar_wait(&pv_done[(i - 1) & 1], ((i - 1) >> 1) & 1, abort_flag, a.status)) { ok = false; continue; }
          tc_fence_after();
#pragma unroll
          for (int u = 0; u < CW / 32; u++) {
            uint32_t rr[32];
            tmem_ld32(tO + lane_off + hs * CW + u * 32, rr);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; j++) rr[j] = __float_as_uint(__uint_as_float(rr[j]) * alpha);
            tmem_st32(tO + lane_off + hs * CW + u * 32, rr);
          }
          tmem_st_wait();
        }
      }
      const float mm = (m_used == -INFINITY) ? 0.f : m_used;
      float sm[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int u = 0; u < CW / 32; u++) {
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          const float p0 = fast_exp2(fmaf(x[u * 32 + 2 * j], c, -mm)), p1 = fast_exp2(fmaf(x[u * 32 + 2 * j + 1], c, -mm));
          const float p2 = fast_exp2(fmaf(x[u * 32 + 2 * j + 2], c, -mm)), p3 = fast_exp2(fmaf(x[u * 32 + 2 * j + 3], c, -mm));
          sm[0] += p0; sm[1] += p1; sm[2] += p2; sm[3] += p3;
          pk[j] = pack_bf16(p0, p1);
          pk[j + 1] = pack_bf16(p2, p3);
        }
        tmem_st16(tS[st] + lane_off + hs * (CW / 2) + u * 16, pk);
      }
      const float sum = (sm[0] + sm[1]) + (sm[2] + sm[3]);
      l += sum;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[st]);
    }
    xl[hs * 128 + r] = l;
    asm volatile("bar.sync %0, %1;" ::"r"(2 + quad), "n"(NS * 32) : "memory");
#pragma unroll
    for (int o = 1; o < NS; o++) l += xl[((hs + o) % NS) * 128 + r];
    if (ok && mbar_wait(&pv_done[(ntile - 1) & 1], ((ntile - 1) >> 1) & 1, abort_flag, a.status)) {
      tc_fence_after();
      const float inv = 1.f / l;
      bf16* o = reinterpret_cast<bf16*>(a.O) + (row0 + q) * a.o_stride + (long long)h * HD;
#pragma unroll
      for (int u = 0; u < CW / 32; u++) {
        const int cc = hs * (CW / 32) + u;
        uint32_t rr[32];
        tmem_ld32(tO + lane_off + cc * 32, rr);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 qv;
            uint32_t* w = reinterpret_cast<uint32_t*>(&qv);
#pragma unroll
            for (int e = 0; e < 4; e++)
              w[e] = pack_bf16(__uint_as_float(rr[j + 2 * e]) * inv, __uint_as_float(rr[j + 2 * e + 1]) * inv);
            *reinterpret_cast<uint4*>(o + cc * 32 + j) = qv;
          }
        }
      }
      if (row_ok && hs == 0) {
        const long long si = ((long long)b * a.H + h) * a.T + q;
        const float ln2 = 0.6931471805599453f;
        if (a.lse) a.lse[si] = (m_used + log2f(l)) * ln2;
        if (a.l) a.l[si] = l;
        if (a.m) a.m[si] = m_used * ln2;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}


// ------------------------------------------------------------------------------------------------------------------
// Persistent forward kernel.  A kernel that allocates tensor memory runs ONE CTA per SM (measured: the runtime reports
// an occupancy of one for any kernel containing tcgen05.alloc, whatever its other resources), so in the kernel above
// every (query tile, head) pays its launch, barrier set-up, tensor-memory allocation, the latency of its first
// loads and its final store with nothing else running on the SM: about as long as five key tiles of work, and a
// query tile of the benchmark (documents of ~512 tokens, windows) sees only three to five key tiles.  Here one CTA
// per SM walks a list of (query tile, head, batch row) items, heaviest first.  The roles are the same as above, but
// they run through the item list asynchronously: the producer is already loading Q, K and V of the next item (Q is
// double-buffered) while the threads finish the current one, the S issuer starts the next item's first products as
// soon as their buffers are free, and only the first P V of an item waits until the threads have taken the previous
// item's O out of tensor memory.
constexpr int PF_SMEM = TILE_BYTES * 6 + 1024 + 256 + 3 * NS * 128 * 4;

__device__ __forceinline__ void pf_item(const AttnArgs& a, int item, int nqt, int& qt, int& h, int& b) {
  // heavy (late) query tiles first; within a query tile all heads and batch rows cost about the same
  const int hb = a.H * a.B;
  qt = nqt - 1 - item / hb;
  const int rem = item % hb;
  h = rem % a.H;
  b = rem / a.H;
}

__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_persistent_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                           const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const FwdParams p,
                           const int nitems, long long* prof) {
  grid_launch_dependents();   // the GEMM that follows may set itself up while this kernel runs (it still waits for our completion)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                    // 2 stages (items)
  uint8_t* sK = smem + 2 * TILE_BYTES;   // 2 stages (tiles)
  uint8_t* sV = smem + 4 * TILE_BYTES;   // 2 stages (tiles)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * TILE_BYTES);
  uint64_t* q_full = bars;        // [2] Q of an item (and its first key tile index) is in place
  uint64_t* q_free = bars + 2;    // [2] every role has taken the item's parameters and its last S has been issued
  uint64_t* k_full = bars + 4;    // [2]
  uint64_t* v_full = bars + 6;    // [2]
  uint64_t* s_full = bars + 8;    // [2] S of a tile is in TMEM; also frees the tile's K stage
  uint64_t* p_ready = bars + 10;  // [2]
  uint64_t* pv_done = bars + 12;  // [2] P V of a tile has been accumulated; also frees its V stage and its S/P buffer
  uint64_t* o_free = bars + 14;   // [1] the threads have read the item's O out of tensor memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* item_jlo = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [2] first key tile of the item in each Q stage
  float* xmax = reinterpret_cast<float*>(smem + 6 * TILE_BYTES + 256);  // [2 parities][NS][128 rows]
  float* xl = xmax + 2 * NS * 128;                                      // [NS][128 rows]

  const AttnArgs& a = p.a;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqt = a.T / BQ;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; i++) {
      mbar_init(&q_full[i], 1); mbar_init(&q_free[i], 1 + NS * 4 + 1);
      mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_ready[i], NS * 4); mbar_init(&pv_done[i], 1);
    }
    mbar_init(o_free, NS * 4);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmO);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS[2] = {tmem_base, tmem_base + 128};
  const uint32_t tO = tmem_base + 256;

  // Every role walks the same items in the same order.  n = number of this CTA's items so far (Q stage n & 1, phase
  // (n >> 1) & 1); tc = number of key tiles so far (K / V / S stage tc & 1, phase (tc >> 1) & 1).
  if (warp == 0) {
    // ---------------- TMA producer (whole warp: the 128 document starts of an item are reduced by the 32 lanes) ----------------
    int tc = 0;
    bool ok = true;
    for (int item = blockIdx.x, n = 0; item < nitems && ok; item += gridDim.x, n++) {
      int qt, h, b;
      pf_item(a, item, nqt, qt, h, b);
      const int kvh = h / (a.H / a.Hkv);
      const int q0 = qt * BQ;
      const long long row0 = (long long)b * a.T;
      const int jhi = (q0 + BQ - 1) / BKV;
      int jlo = max(0, q0 - a.window_left) / BKV;
      if (a.doc_start) {
        // key tiles that lie before the earliest document start of these 128 queries are fully masked
        const int4 v = *reinterpret_cast<const int4*>(a.doc_start + row0 + q0 + lane * 4);
        const int mn = __reduce_min_sync(0xffffffffu, min(min(v.x, v.y), min(v.z, v.w)));
        jlo = max(jlo, mn / BKV);
      }
      const int ntile = jhi - jlo + 1;
      if (lane == 0) {
        const int qs = n & 1;
        if (n >= 2 && !mbar_wait(&q_free[qs], ((n - 2) >> 1) & 1, abort_flag, a.status)) ok = false;
        if (ok) {
          item_jlo[qs] = jlo;
          mbar_expect_tx(&q_full[qs], TILE_BYTES);   // the arrive publishes item_jlo to the roles that wait on q_full
          tma_load_2d(sQ + qs * TILE_BYTES, &tmQ, &q_full[qs], p.q_col0 + h * HD, (int)(row0 + q0));
          tma_load_2d(sQ + qs * TILE_BYTES + TILE_BYTES / 2, &tmQ, &q_full[qs], p.q_col0 + h * HD + 64, (int)(row0 + q0));
          for (int i = 0; i < ntile; i++, tc++) {
            const int st = tc & 1;
            const uint32_t ph2 = ((tc - 2) >> 1) & 1;   // phase of tile tc-2, the previous user of this stage
            const int krow = (int)(row0 + (jlo + i) * BKV);
            if (tc >= 2 && !mbar_wait(&s_full[st], ph2, abort_flag, a.status)) { ok = false; break; }
            mbar_expect_tx(&k_full[st], TILE_BYTES);
            tma_load_2d(sK + st * TILE_BYTES, &tmK, &k_full[st], p.k_col0 + kvh * HD, krow);
            tma_load_2d(sK + st * TILE_BYTES + TILE_BYTES / 2, &tmK, &k_full[st], p.k_col0 + kvh * HD + 64, krow);
            if (tc >= 2 && !mbar_wait(&pv_done[st], ph2, abort_flag, a.status)) { ok = false; break; }
            mbar_expect_tx(&v_full[st], TILE_BYTES);
            tma_load_2d(sV + st * TILE_BYTES, &tmV, &v_full[st], p.v_col0 + kvh * HD, krow);
            tma_load_2d(sV + st * TILE_BYTES + TILE_BYTES / 2, &tmV, &v_full[st], p.v_col0 + kvh * HD + 64, krow);
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      tc = __shfl_sync(0xffffffffu, tc, 0);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- S = Q K^T issuer ----------------
      constexpr uint32_t idesc_s = idesc_bf16(BQ, BKV, false, false);  // both operands K-major
      int tc = 0;
      bool ok = true;
      Cyc cy;   // laps: 0 waiting (Q, K, free S buffer), 1 issuing
      cy.start();
      for (int item = blockIdx.x, n = 0; item < nitems && ok; item += gridDim.x, n++) {
        int qt, h, b;
        pf_item(a, item, nqt, qt, h, b);
        const int qs = n & 1;
        if (!mbar_wait(&q_full[qs], (n >> 1) & 1, abort_flag, a.status)) break;
        const int ntile = (qt * BQ + BQ - 1) / BKV - item_jlo[qs] + 1;
        const uint32_t q_addr = smem_u32(sQ + qs * TILE_BYTES);
        for (int i = 0; i < ntile; i++, tc++) {
          const int st = tc & 1;
          if (!mbar_wait(&k_full[st], (tc >> 1) & 1, abort_flag, a.status)) { ok = false; break; }
          // S overwrites the buffer that held P of tile tc-2: its P V must have been executed
          if (tc >= 2 && !mbar_wait(&pv_done[st], ((tc - 2) >> 1) & 1, abort_flag, a.status)) { ok = false; break; }
          tc_fence_after();
          cy.lap(0);
          const uint32_t k_addr = smem_u32(sK + st * TILE_BYTES);
#pragma unroll
          for (int k = 0; k < HD / 16; k++) {
            const uint32_t off = (k >> 2) * (TILE_BYTES / 2) + (k & 3) * 32;
            mma_ss(tS[st], smem_desc_sw128(q_addr + off, 16, 1024), smem_desc_sw128(k_addr + off, 16, 1024), idesc_s, k > 0);
          }
          tc_commit(&s_full[st]);
          cy.lap(1);
        }
        if (ok) tc_commit(&q_free[qs]);   // the item's last S has been issued: its Q stage may be refilled once it completes
      }
      cy.store(prof, 1, tc);
    }
  } else if (warp == 2) {
    if (lane == 0) {
      // ---------------- O += P V issuer ----------------
      constexpr uint32_t idesc_o = idesc_bf16(BQ, HD, false, true);    // V is N-contiguous
      int tc = 0;
      bool ok = true;
      Cyc cy;   // laps: 0 waiting (Q, P, V, free O), 1 issuing
      cy.start();
      for (int item = blockIdx.x, n = 0; item < nitems && ok; item += gridDim.x, n++) {
        int qt, h, b;
        pf_item(a, item, nqt, qt, h, b);
        const int qs = n & 1;
        if (!mbar_wait(&q_full[qs], (n >> 1) & 1, abort_flag, a.status)) break;
        const int ntile = (qt * BQ + BQ - 1) / BKV - item_jlo[qs] + 1;
        mbar_arrive(&q_free[qs]);
        // the accumulator still holds the previous item's O until the threads have read it
        if (n >= 1 && !mbar_wait(o_free, (n - 1) & 1, abort_flag, a.status)) break;
        for (int i = 0; i < ntile; i++, tc++) {
          const int st = tc & 1;
          const uint32_t ph = (tc >> 1) & 1;
          if (!mbar_wait(&p_ready[st], ph, abort_flag, a.status)) { ok = false; break; }
          if (!mbar_wait(&v_full[st], ph, abort_flag, a.status)) { ok = false; break; }
          tc_fence_after();
          cy.lap(0);
          const uint32_t v_addr = smem_u32(sV + st * TILE_BYTES);
#pragma unroll
          for (int k = 0; k < BKV / 16; k++)
            mma_ts(tO, tS[st] + k * 8, smem_desc_sw128(v_addr + k * 2048, TILE_BYTES / 2, 1024), idesc_o, (i > 0 || k > 0) ? 1u : 0u);
          tc_commit(&pv_done[st]);
          cy.lap(1);
        }
      }
      cy.store(prof, 2, tc);
    }
  } else if (warp >= 4) {
    // ---------------- softmax: NS threads per query row, each owns CW = 128 / NS of the keys of a tile ----------------
    const int quad = warp & 3;
    const int hs = (warp - 4) >> 2;        // which CW keys of each tile
    const int r = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const float c = rsqrtf((float)HD) * LOG2E;
    int tc = 0;
    bool ok = true;
    Cyc cy;   // laps: 0 waiting for S (and Q), 1 S load + masks + maximum, 2 exchange barrier, 3 rescale, 4 exponentials + P store, 5 arrive, 6 end of item
    cy.start();
    for (int item = blockIdx.x, n = 0; item < nitems; item += gridDim.x, n++) {
      int qt, h, b;
      pf_item(a, item, nqt, qt, h, b);
      const int qs = n & 1;
      const int q0 = qt * BQ;
      const int q = q0 + r;
      const long long row0 = (long long)b * a.T;
      // After a timed-out wait a warp keeps walking the items and tiles (skipping the work) so that it still meets
      // its partner warp at every row barrier; both read the same tile count from shared memory.
      if (ok && !mbar_wait(&q_full[qs], (n >> 1) & 1, abort_flag, a.status)) ok = false;
      const int jlo = item_jlo[qs];
      const int ntile = min(max((q0 + BQ - 1) / BKV - jlo + 1, 0), nqt);
      __syncwarp();
      // The Q stage of the PREVIOUS item doubles as the staging area of that item's O (see the end of the item):
      // it goes back to the producer once the store has read it.
      if (ok && lane == 0 && n >= 1) { bulk_wait_read<0>(); mbar_arrive(&q_free[(n - 1) & 1]); }
      int lo = max(0, q - a.window_left);
      if (a.doc_start) lo = max(lo, a.doc_start[row0 + q]);
      float m_used = -INFINITY, l = 0.f;
      for (int i = 0; i < ntile; i++, tc++) {
        const int st = tc & 1;
        const uint32_t ph = (tc >> 1) & 1;
        const int k0 = (jlo + i) * BKV + hs * CW;
        // After a timed-out wait the warp keeps walking the loop (skipping the work) so that it still
        // meets its partner warps at every row barrier.
        if (ok && !mbar_wait(&s_full[st], ph, abort_flag, a.status)) ok = false;
        if (!ok) { asm volatile("bar.sync %0, %1;" ::"r"(2 + quad), "n"(NS * 32) : "memory"); continue; }
        tc_fence_after();
        cy.lap(0);
        float x[CW];
#pragma unroll
        for (int u = 0; u < CW / 32; u++)
          tmem_ld32(tS[st] + lane_off + hs * CW + u * 32, *reinterpret_cast<uint32_t(*)[32]>(&x[u * 32]));
        tmem_ld_wait();
        const bool need_mask = (k0 + CW - 1 > q) || (k0 < lo);
        if (need_mask) {
#pragma unroll
          for (int j = 0; j < CW; j++) {
            const int k = k0 + j;
            x[j] = (k <= q && k >= lo) ? x[j] : -INFINITY;
          }
        }
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < CW; j += 4) {
          mx[0] = fmaxf(mx[0], x[j]); mx[1] = fmaxf(mx[1], x[j + 1]);
          mx[2] = fmaxf(mx[2], x[j + 2]); mx[3] = fmaxf(mx[3], x[j + 3]);
        }
        float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * c;
        xmax[(tc & 1) * (NS * 128) + hs * 128 + r] = mt;
        cy.lap(1);
        asm volatile("bar.sync %0, %1;" ::"r"(2 + quad), "n"(NS * 32) : "memory");
        cy.lap(2);
#pragma unroll
        for (int o = 1; o < NS; o++) mt = fmaxf(mt, xmax[(tc & 1) * (NS * 128) + ((hs + o) % NS) * 128 + r]);
        const bool grow = mt > m_used + 8.f || (m_used == -INFINITY && mt > -INFINITY);
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = fmaxf(m_used, mt);
          const float alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new);
          l *= alpha;
          m_used = m_new;
          if (i > 0) {
            // O lives in TMEM and is being accumulated by the tensor core: wait for the previous tile's P V
            if (!mbar_wait(&pv_done[(tc - 1) & 1], ((tc - 1) >> 1) & 1, abort_flag, a.status)) { ok = false; continue; }
            tc_fence_after();
#pragma unroll
            for (int u = 0; u < CW / 32; u++) {
              uint32_t rr[32];
              tmem_ld32(tO + lane_off + hs * CW + u * 32, rr);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; j++) rr[j] = __float_as_uint(__uint_as_float(rr[j]) * alpha);
              tmem_st32(tO + lane_off + hs * CW + u * 32, rr);
            }
            tmem_st_wait();
          }
        }
        cy.lap(3);
        const float mm = (m_used == -INFINITY) ? 0.f : m_used;
        float sm[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int u = 0; u < CW / 32; u++) {
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const float p0 = fast_exp2(fmaf(x[u * 32 + 2 * j], c, -mm)), p1 = fast_exp2(fmaf(x[u * 32 + 2 * j + 1], c, -mm));
            const float p2 = fast_exp2(fmaf(x[u * 32 + 2 * j + 2], c, -mm)), p3 = fast_exp2(fmaf(x[u * 32 + 2 * j + 3], c, -mm));
            sm[0] += p0; sm[1] += p1; sm[2] += p2; sm[3] += p3;
            pk[j] = pack_bf16(p0, p1);
            pk[j + 1] = pack_bf16(p2, p3);
          }
          tmem_st16(tS[st] + lane_off + hs * (CW / 2) + u * 16, pk);
        }
        l += (sm[0] + sm[1]) + (sm[2] + sm[3]);
        cy.lap(4);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[st]);
        cy.lap(5);
      }
      // ---- the item's O: out of tensor memory first (so that the next item's products can start), then to global memory ----
      xl[hs * 128 + r] = l;
      asm volatile("bar.sync %0, %1;" ::"r"(2 + quad), "n"(NS * 32) : "memory");
#pragma unroll
      for (int o = 1; o < NS; o++) l += xl[((hs + o) % NS) * 128 + r];
      if (ok && !mbar_wait(&pv_done[(tc - 1) & 1], ((tc - 1) >> 1) & 1, abort_flag, a.status)) ok = false;
      if (ok) {
        tc_fence_after();
        uint32_t rr[CW / 32][32];
#pragma unroll
        for (int u = 0; u < CW / 32; u++) tmem_ld32(tO + lane_off + (hs * (CW / 32) + u) * 32, rr[u]);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(o_free);
        const float inv = 1.f / l;
        // This warp's 32 rows x 64 columns of O leave through shared memory and ONE tiled TMA store (whole 128-byte
        // lines; sixteen-byte stores of one row per lane cost every store instruction 32 separate lines).  The
        // staging area is the item's own Q stage: every S product of the item has been executed (the threads have
        // consumed the last S), and the stage is handed back to the producer only after the store has read it.
        uint8_t* stage = sQ + qs * TILE_BYTES + (warp - 4) * 4096;
#pragma unroll
        for (int u = 0; u < CW / 32; u++) {
#pragma unroll
          for (int j = 0; j < 4; j++) {
            uint4 qv;
            uint32_t* w = reinterpret_cast<uint32_t*>(&qv);
#pragma unroll
            for (int e = 0; e < 4; e++)
              w[e] = pack_bf16(__uint_as_float(rr[u][8 * j + 2 * e]) * inv, __uint_as_float(rr[u][8 * j + 2 * e + 1]) * inv);
            *reinterpret_cast<uint4*>(stage + lane * 128 + (((u * 4 + j) ^ (lane & 7)) << 4)) = qv;
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(&tmO, stage, h * HD + hs * CW, (int)(row0 + q0 + quad * 32), 0);
          bulk_commit();
        }
        if (hs == 0) {
          const long long si = ((long long)b * a.H + h) * a.T + q;
          const float ln2 = 0.6931471805599453f;
          if (a.lse) a.lse[si] = (m_used + log2f(l)) * ln2;
          if (a.l) a.l[si] = l;
          if (a.m) a.m[si] = m_used * ln2;
        }
      }
      // the row's partner reads xl of this item before either thread may overwrite it for the next one
      asm volatile("bar.sync %0, %1;" ::"r"(2 + quad), "n"(NS * 32) : "memory");
      cy.lap(6);
    }
    if (lane == 0) { bulk_wait_all(); cy.store(prof, warp, tc); }   // the last item's store has left shared memory
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}


// ------------------------------------------------------------------------------------------------------------------
// Two query tiles per CTA in ping-pong.  In the kernels above the two threads of a query row work on the same S
// tile, meet at a barrier to exchange their maxima and therefore run their phases in lockstep: while they load S and
// take the maximum the special-function unit idles, while they evaluate 2^x nothing else of theirs can run, and the
// tensor pipe waits for P.  Here one CTA owns TWO 128-query tiles X = A, B that read the same keys and values: the two
// query heads of one key/value head at the same positions (grouped-query attention with an even group), or two
// adjacent query tiles of one head.  Tensor memory holds S_A, S_B (P overwrites S in place as bf16) and O_A, O_B,
// 128 columns each.  One thread owns one query row (no exchange between threads, no barrier per tile) in one of two
// softmax warpgroups, and one thread issues every product in the order
//     S_A(0) S_B(0)   { O_A += P_A(j) V(j);  S_A(j+1);  O_B += P_B(j) V(j);  S_B(j+1) }  j = 0, 1, ...
// so that the softmax of one tile runs while the tensor pipe works for the other, and every K / V tile is loaded once
// for both.  A thread reads its row of S twice from tensor memory (maximum, then exponentials; 64 columns at a time)
// instead of holding 128 values in registers.  Persistent: one CTA per SM walks the items, heaviest first.
constexpr int PP_SMEM = TILE_BYTES * 6 + 1024 + 512;

struct PairItem {
  int qt[2], h[2], b, kvh;
  bool valid_b;
};
__device__ __forceinline__ PairItem pp_item(const AttnArgs& a, int item, int nqt, bool gqa) {
  PairItem it;
  if (gqa) {   // heads 2g and 2g+1 of one key/value head, same query tile
    const int per = (a.H / 2) * a.B;
    const int qt = nqt - 1 - item / per, rem = item % per;
    const int hp = rem % (a.H / 2);
    it.b = rem / (a.H / 2);
    it.qt[0] = it.qt[1] = qt;
    it.h[0] = 2 * hp; it.h[1] = 2 * hp + 1;
    it.valid_b = true;
  } else {     // query tiles 2p and 2p+1 of one head
    const int per = a.H * a.B;
    const int qp = (nqt + 1) / 2 - 1 - item / per, rem = item % per;
    it.b = rem / a.H;
    it.h[0] = it.h[1] = rem % a.H;
    it.qt[0] = 2 * qp; it.qt[1] = 2 * qp + 1;
    it.valid_b = it.qt[1] < nqt;
  }
  it.kvh = it.h[0] / (a.H / a.Hkv);
  return it;
}

__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const FwdParams p, const int nitems, const int gqa, long long* prof) {
  grid_launch_dependents();   // the GEMM that follows may set itself up while this kernel runs (it still waits for our completion)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                    // Q_A, Q_B
  uint8_t* sK = smem + 2 * TILE_BYTES;   // 2 stages
  uint8_t* sV = smem + 4 * TILE_BYTES;   // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * TILE_BYTES);
  uint64_t* q_full = bars;          // both Q tiles and the item's key ranges are in place
  uint64_t* q_free = bars + 1;      // the item's last S has been executed and every softmax warp has read the ranges
  uint64_t* k_full = bars + 2;      // [2]
  uint64_t* v_full = bars + 4;      // [2]
  uint64_t* k_free = bars + 6;      // [2] both S products of the stage's tile have been executed
  uint64_t* v_free = bars + 8;      // [2] both P V products of the stage's tile have been executed
  uint64_t* s_full = bars + 10;     // [2: A, B]
  uint64_t* p_ready = bars + 12;    // [2: A, B]
  uint64_t* pv_done = bars + 14;    // [2: A, B]
  uint64_t* o_free = bars + 16;     // [2: A, B] the warpgroup has read the item's O out of tensor memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* rng = reinterpret_cast<volatile int*>(tmem_slot + 2);   // jlo_A, jhi_A, jlo_B, jhi_B of the item in sQ

  const AttnArgs& a = p.a;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqt = a.T / BQ;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(q_free, 1 + 8);
    for (int i = 0; i < 2; i++) {
      mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1); mbar_init(&k_free[i], 1); mbar_init(&v_free[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_ready[i], 4); mbar_init(&pv_done[i], 1); mbar_init(&o_free[i], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Every role walks the same items in the same order.  n = items of this CTA so far (phase n & 1 of q_full / q_free);
  // tu = key tiles loaded so far (K / V stage tu & 1, phase (tu >> 1) & 1); tcX = key tiles tile X has processed so
  // far (phase tcX & 1 of s_full / p_ready / pv_done [X]); nX = items in which X had any key tile (o_free[X]).
  if (warp < 4) {
  if (warp == 0) {
    // ---------------- TMA producer (whole warp: the document starts of a query tile are reduced by the 32 lanes) ----------------
    int tu = 0;
    bool ok = true;
    for (int item = blockIdx.x, n = 0; item < nitems && ok; item += gridDim.x, n++) {
      const PairItem it = pp_item(a, item, nqt, gqa != 0);
      const long long row0 = (long long)it.b * a.T;
      int jlo[2], jhi[2];
#pragma unroll
      for (int X = 0; X < 2; X++) {
        const int q0 = it.qt[X] * BQ;
        jhi[X] = it.qt[X];
        jlo[X] = max(0, q0 - a.window_left) / BKV;
        if (a.doc_start && (X == 0 || it.valid_b)) {
          // key tiles that lie before the earliest document start of these 128 queries are fully masked
          const int4 v = *reinterpret_cast<const int4*>(a.doc_start + row0 + q0 + lane * 4);
          const int mn = __reduce_min_sync(0xffffffffu, min(min(v.x, v.y), min(v.z, v.w)));
          jlo[X] = max(jlo[X], mn / BKV);
        }
      }
      if (!it.valid_b) { jlo[1] = 1; jhi[1] = 0; }
      const int jmin = it.valid_b ? min(jlo[0], jlo[1]) : jlo[0];
      const int jmax = it.valid_b ? max(jhi[0], jhi[1]) : jhi[0];
      const int nu = jmax - jmin + 1;
      if (lane == 0) {
        if (n >= 1 && !mbar_wait(q_free, (n - 1) & 1, abort_flag, a.status)) ok = false;
        if (ok) {
          rng[0] = jlo[0]; rng[1] = jhi[0]; rng[2] = jlo[1]; rng[3] = jhi[1];
          mbar_expect_tx(q_full, it.valid_b ? 2 * TILE_BYTES : TILE_BYTES);   // the arrive publishes rng
#pragma unroll
          for (int X = 0; X < 2; X++) {
            if (X == 1 && !it.valid_b) break;
            const int qrow = (int)(row0 + it.qt[X] * BQ);
            tma_load_2d(sQ + X * TILE_BYTES, &tmQ, q_full, p.q_col0 + it.h[X] * HD, qrow);
            tma_load_2d(sQ + X * TILE_BYTES + TILE_BYTES / 2, &tmQ, q_full, p.q_col0 + it.h[X] * HD + 64, qrow);
          }
          for (int u = 0; u < nu; u++, tu++) {
            const int st = tu & 1;
            const uint32_t ph2 = ((tu - 2) >> 1) & 1;   // phase of tile tu-2, the previous user of this stage
            const int krow = (int)(row0 + (jmin + u) * BKV);
            if (tu >= 2 && !mbar_wait(&k_free[st], ph2, abort_flag, a.status)) { ok = false; break; }
            mbar_expect_tx(&k_full[st], TILE_BYTES);
            tma_load_2d(sK + st * TILE_BYTES, &tmK, &k_full[st], p.k_col0 + it.kvh * HD, krow);
            tma_load_2d(sK + st * TILE_BYTES + TILE_BYTES / 2, &tmK, &k_full[st], p.k_col0 + it.kvh * HD + 64, krow);
            if (tu >= 2 && !mbar_wait(&v_free[st], ph2, abort_flag, a.status)) { ok = false; break; }
            mbar_expect_tx(&v_full[st], TILE_BYTES);
            tma_load_2d(sV + st * TILE_BYTES, &tmV, &v_full[st], p.v_col0 + it.kvh * HD, krow);
            tma_load_2d(sV + st * TILE_BYTES + TILE_BYTES / 2, &tmV, &v_full[st], p.v_col0 + it.kvh * HD + 64, krow);
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      tu = __shfl_sync(0xffffffffu, tu, 0);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- the one issuer of every product ----------------
      constexpr uint32_t idesc_s = idesc_bf16(BQ, BKV, false, false);  // both operands K-major
      constexpr uint32_t idesc_o = idesc_bf16(BQ, HD, false, true);    // V is N-contiguous
      int tu = 0, tcx[2] = {0, 0}, nx[2] = {0, 0};
      bool ok = true;
      Cyc cy;   // laps: 0 waiting (Q, K, V, P_A, P_B, free O), 1 issuing
      cy.start();
      for (int item = blockIdx.x, n = 0; item < nitems && ok; item += gridDim.x, n++) {
        if (!mbar_wait(q_full, n & 1, abort_flag, a.status)) break;
        const int jlo[2] = {rng[0], rng[2]}, jhi[2] = {rng[1], rng[3]};
        const bool has[2] = {jlo[0] <= jhi[0], jlo[1] <= jhi[1]};
        const int jmin = has[1] ? min(jlo[0], jlo[1]) : jlo[0];
        const int jmax = has[1] ? max(jhi[0], jhi[1]) : jhi[0];
        const int nu = jmax - jmin + 1;
        auto in = [&](int X, int u) { const int j = jmin + u; return j >= jlo[X] && j <= jhi[X]; };
        auto issue_s = [&](int X, int st) {
          const uint32_t q_addr = smem_u32(sQ + X * TILE_BYTES), k_addr = smem_u32(sK + st * TILE_BYTES);
#pragma unroll
          for (int k = 0; k < HD / 16; k++) {
            const uint32_t off = (k >> 2) * (TILE_BYTES / 2) + (k & 3) * 32;
            mma_ss(tmem_base + X * 128, smem_desc_sw128(q_addr + off, 16, 1024), smem_desc_sw128(k_addr + off, 16, 1024), idesc_s, k > 0);
          }
          tc_commit(&s_full[X]);
        };
        bool first[2] = {true, true};   // X's next P V is the first of the item: it overwrites O_X
        // first key tile of the item
        if (!mbar_wait(&k_full[tu & 1], (tu >> 1) & 1, abort_flag, a.status)) break;
        tc_fence_after();
        cy.lap(0);
        if (in(0, 0)) issue_s(0, tu & 1);
        if (in(1, 0)) issue_s(1, tu & 1);
        tc_commit(&k_free[tu & 1]);
        if (nu == 1) tc_commit(q_free);
        cy.lap(1);
        for (int u = 0; u < nu && ok; u++) {
          const int st = (tu + u) & 1, st1 = (tu + u + 1) & 1;
          const uint32_t ph = ((tu + u) >> 1) & 1, ph1 = ((tu + u + 1) >> 1) & 1;
          bool v_seen = false, k_seen = false;
#pragma unroll
          for (int X = 0; X < 2; X++) {
            if (in(X, u)) {
              if (!mbar_wait(&p_ready[X], tcx[X] & 1, abort_flag, a.status)) { ok = false; break; }
              if (!v_seen && !mbar_wait(&v_full[st], ph, abort_flag, a.status)) { ok = false; break; }
              v_seen = true;
              // O_X still holds the previous item's result until its warpgroup has read it
              if (first[X] && nx[X] >= 1 && !mbar_wait(&o_free[X], (nx[X] - 1) & 1, abort_flag, a.status)) { ok = false; break; }
              tc_fence_after();
              cy.lap(0);
              const uint32_t v_addr = smem_u32(sV + st * TILE_BYTES);
#pragma unroll
              for (int k = 0; k < BKV / 16; k++)
                mma_ts(tmem_base + 256 + X * 128, tmem_base + X * 128 + k * 8, smem_desc_sw128(v_addr + k * 2048, TILE_BYTES / 2, 1024),
                       idesc_o, (!first[X] || k > 0) ? 1u : 0u);
              tc_commit(&pv_done[X]);
              first[X] = false;
              tcx[X]++;
              cy.lap(1);
            }
            if (X == 1) tc_commit(&v_free[st]);
            if (u + 1 < nu) {
              if (in(X, u + 1)) {
                if (!k_seen && !mbar_wait(&k_full[st1], ph1, abort_flag, a.status)) { ok = false; break; }
                k_seen = true;
                tc_fence_after();
                cy.lap(0);
                issue_s(X, st1);
                cy.lap(1);
              }
              if (X == 1) {
                tc_commit(&k_free[st1]);
                if (u + 1 == nu - 1) tc_commit(q_free);   // the item's last S: Q may be replaced once it has been executed
              }
            }
          }
        }
        tu += nu;
        if (has[0]) nx[0]++;
        if (has[1]) nx[1]++;
      }
      cy.store(prof, 1, tu);
    }
  }
  } else {
    // ---------------- softmax warpgroups: X = 0 (warps 4-7) and 1 (warps 8-11), one thread per query row ----------------
    const int X = (warp - 4) >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const uint32_t tS = tmem_base + X * 128 + lane_off, tO = tmem_base + 256 + X * 128 + lane_off;
    const float c = rsqrtf((float)HD) * LOG2E;
    const uint64_t c2 = pack2(c, c);
    int tc = 0, nX = 0;
    bool ok = true;
    Cyc cy;   // laps: 0 waiting for S (and Q), 1 pass 1 (S load, masks, maximum), 3 rescale, 4 pass 2 (S load, exponentials, P store), 5 arrive, 6 end of item
    cy.start();
    for (int item = blockIdx.x, n = 0; item < nitems && ok; item += gridDim.x, n++) {
      const PairItem it = pp_item(a, item, nqt, gqa != 0);
      if (!mbar_wait(q_full, n & 1, abort_flag, a.status)) break;
      const int jlo = rng[2 * X], jhi = rng[2 * X + 1];
      __syncwarp();
      if (lane == 0) mbar_arrive(q_free);
      if (jlo > jhi) continue;
      const int q = it.qt[X] * BQ + r, h = it.h[X];
      const long long row0 = (long long)it.b * a.T;
      int lo = max(0, q - a.window_left);
      if (a.doc_start) lo = max(lo, a.doc_start[row0 + q]);
      float m_used = -INFINITY, l = 0.f;
      for (int j = jlo; j <= jhi; j++, tc++) {
        const int k0 = j * BKV;
        if (!mbar_wait(&s_full[X], tc & 1, abort_flag, a.status)) { ok = false; break; }
        tc_fence_after();
        cy.lap(0);
        // Masks.  The keys this row may see in the tile are the columns ca..cb.  Per group of 32 columns the warp
        // decides together: every lane sees all of it (no work), no lane sees any of it (P = 0, no exponentials), or
        // mixed (element-wise select).  On a diagonal tile one group of four is mixed and those right of it are empty.
        const int ca = max(lo - k0, 0), cb = min(q - k0, BKV - 1);
        const bool any_mask = __any_sync(0xffffffffu, ca > 0 || cb < BKV - 1);
        unsigned empty = 0, mixed = 0;   // bit g: no lane of the warp sees a key of group g / some do, some do not
        if (any_mask) {
#pragma unroll
          for (int g = 0; g < 4; g++) {
            const bool all_in = __all_sync(0xffffffffu, ca <= g * 32 && cb >= g * 32 + 31);
            const bool none_in = __all_sync(0xffffffffu, cb < g * 32 || ca > g * 32 + 31);
            if (none_in) empty |= 1u << g;
            else if (!all_in) mixed |= 1u << g;
          }
        }
        // ---- pass 1: the row maximum (three-input maxima, four chains), 64 columns at a time ----
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
          if (((empty >> (2 * hf)) & 3u) == 3u) continue;
          float x[64];
          tmem_ld32(tS + hf * 64, *reinterpret_cast<uint32_t(*)[32]>(&x[0]));
          tmem_ld32(tS + hf * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&x[32]));
          tmem_ld_wait();
#pragma unroll
          for (int gg = 0; gg < 2; gg++) {
            const int g = 2 * hf + gg;
            if (empty & (1u << g)) continue;
            if (mixed & (1u << g)) {
#pragma unroll
              for (int e = 0; e < 32; e++) x[gg * 32 + e] = (g * 32 + e >= ca && g * 32 + e <= cb) ? x[gg * 32 + e] : -INFINITY;
            }
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              mx[0] = max3(mx[0], x[gg * 32 + e], x[gg * 32 + e + 1]); mx[1] = max3(mx[1], x[gg * 32 + e + 2], x[gg * 32 + e + 3]);
              mx[2] = max3(mx[2], x[gg * 32 + e + 4], x[gg * 32 + e + 5]); mx[3] = max3(mx[3], x[gg * 32 + e + 6], x[gg * 32 + e + 7]);
            }
          }
        }
        const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * c;
        cy.lap(1);
        const bool grow = mt > m_used + 8.f || (m_used == -INFINITY && mt > -INFINITY);
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = fmaxf(m_used, mt);
          const float alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new);
          l *= alpha;
          m_used = m_new;
          if (j > jlo) {
            // O_X is being accumulated by the tensor core: wait for the previous tile's P V, then rescale the row
            if (!mbar_wait(&pv_done[X], (tc - 1) & 1, abort_flag, a.status)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int u = 0; u < 4; u++) {
              uint32_t rr[32];
              tmem_ld32(tO + u * 32, rr);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 32; e++) rr[e] = __float_as_uint(__uint_as_float(rr[e]) * alpha);
              tmem_st32(tO + u * 32, rr);
            }
            tmem_st_wait();
          }
        }
        cy.lap(3);
        // ---- pass 2: P = 2^(c S - m) as bf16 over S, and the row sum; two elements per fma / add ----
        const float mm = (m_used == -INFINITY) ? 0.f : m_used;
        const uint64_t nm2 = pack2(-mm, -mm);
        uint64_t sm2[2] = {0ull, 0ull};   // (+0, +0)
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
          float x[64];
          if (((empty >> (2 * hf)) & 3u) != 3u) {
            tmem_ld32(tS + hf * 64, *reinterpret_cast<uint32_t(*)[32]>(&x[0]));
            tmem_ld32(tS + hf * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&x[32]));
            tmem_ld_wait();
          }
#pragma unroll
          for (int gg = 0; gg < 2; gg++) {
            const int g = 2 * hf + gg;
            uint32_t pk[16];
            if (empty & (1u << g)) {
#pragma unroll
              for (int e = 0; e < 16; e++) pk[e] = 0u;
            } else {
              if (mixed & (1u << g)) {
#pragma unroll
                for (int e = 0; e < 32; e++) x[gg * 32 + e] = (g * 32 + e >= ca && g * 32 + e <= cb) ? x[gg * 32 + e] : -INFINITY;
              }
#pragma unroll
              for (int e = 0; e < 16; e += 2) {
                const int i0 = gg * 32 + 2 * e;
                float t0, t1, t2, t3;
                unpack2(fma2(pack2(x[i0], x[i0 + 1]), c2, nm2), t0, t1);
                unpack2(fma2(pack2(x[i0 + 2], x[i0 + 3]), c2, nm2), t2, t3);
                const float p0 = fast_exp2(t0), p1 = fast_exp2(t1), p2 = fast_exp2(t2), p3 = fast_exp2(t3);
                sm2[0] = add2(sm2[0], pack2(p0, p1));
                sm2[1] = add2(sm2[1], pack2(p2, p3));
                pk[e] = pack_bf16(p0, p1);
                pk[e + 1] = pack_bf16(p2, p3);
              }
            }
            // keys g*32 .. g*32+31 as bf16: 16 columns starting at column g*16.  They overwrite S columns that this
            // thread has already loaded (first half) or no longer needs.
            tmem_st16(tS + g * 16, pk);
          }
        }
        {
          float s0, s1, s2, s3;
          unpack2(sm2[0], s0, s1);
          unpack2(sm2[1], s2, s3);
          l += (s0 + s1) + (s2 + s3);
        }
        cy.lap(4);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[X]);
        cy.lap(5);
      }
      if (!ok) break;
      // ---- the item's O: out of tensor memory (then the next item's P V may start), scaled, to global memory ----
      if (!mbar_wait(&pv_done[X], (tc - 1) & 1, abort_flag, a.status)) break;
      tc_fence_after();
      {
        const float inv = 1.f / l;
        bf16* o = reinterpret_cast<bf16*>(a.O) + (row0 + q) * a.o_stride + (long long)h * HD;
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
          uint32_t rr[2][32];
          tmem_ld32(tO + hf * 64, rr[0]);
          tmem_ld32(tO + hf * 64 + 32, rr[1]);
          tmem_ld_wait();
          if (hf == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&o_free[X]);
          }
#pragma unroll
          for (int u = 0; u < 2; u++) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint4 qv;
              uint32_t* w = reinterpret_cast<uint32_t*>(&qv);
#pragma unroll
              for (int t = 0; t < 4; t++)
                w[t] = pack_bf16(__uint_as_float(rr[u][e + 2 * t]) * inv, __uint_as_float(rr[u][e + 2 * t + 1]) * inv);
              *reinterpret_cast<uint4*>(o + hf * 64 + u * 32 + e) = qv;
            }
          }
        }
      }
      {
        const long long si = ((long long)it.b * a.H + h) * a.T + q;
        const float ln2 = 0.6931471805599453f;
        if (a.lse) a.lse[si] = (m_used + log2f(l)) * ln2;
        if (a.l) a.l[si] = l;
        if (a.m) a.m[si] = m_used * ln2;
      }
      nX++;
      cy.lap(6);
    }
    if (lane == 0) cy.store(prof, warp, tc);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

bool attention_tc_supported(const AttnArgs& a) {
  if (a.hd != HD) return false;
  if (a.T % BQ != 0 || a.T > 8192) return false;  // the dK/dV kernel lists at most 64 query tiles
  if ((a.q_stride & 7) || (a.kv_stride & 7) || (a.o_stride & 7)) return false;
  if (!aligned16(a.Q) || !aligned16(a.K) || !aligned16(a.V) || !aligned16(a.O)) return false;
  if (a.H % a.Hkv != 0) return false;
  if (a.doc_start && !aligned16(a.doc_start)) return false;
  return true;
}

// Cycle accounting (see Cyc): a 16 x 16 table of counters, one row per warp, printed after the launch.
#ifdef FEMTO_ATTN_CYCLES
static long long* g_cycles = nullptr;
static long long* cycles_buffer() {
  static int want = -1;
  if (want < 0) {
    want = getenv("FEMTO_ATTN_PROF") ? 1 : 0;
    if (want && cudaMalloc(&g_cycles, 16 * 16 * sizeof(long long)) != cudaSuccess) g_cycles = nullptr;
  }
  if (g_cycles) cudaMemset(g_cycles, 0, 16 * 16 * sizeof(long long));
  return g_cycles;
}
static void cycles_report(const char* issuers, const char* softmax, int first_issuer, int last_issuer) {
  if (!g_cycles) return;
  cudaDeviceSynchronize();
  long long h[16 * 16];
  cudaMemcpy(h, g_cycles, sizeof(h), cudaMemcpyDeviceToHost);
  printf("cycles of CTA 0 | %s | %s\n", issuers, softmax);
  for (int w = 0; w < 12; w++) {
    if (!((w >= first_issuer && w <= last_issuer) || w == 4 || w == 8)) continue;
    printf("  warp %2d tiles %lld:", w, h[w * 16 + 10]);
    for (int i = 0; i < 7; i++) printf(" %lld", h[w * 16 + i]);
    printf("\n");
  }
  fflush(stdout);
}
#else
static long long* cycles_buffer() { return nullptr; }
static void cycles_report(const char*, const char*, int, int) {}
#endif

int attention_fwd_tc(const AttnArgs& a, cudaStream_t s) {
  if (!attention_tc_supported(a)) return femto_fail(FEMTO_ERR_UNSUPPORTED, "attention_fwd_tc: unsupported shape");
  const long long N = (long long)a.B * a.T;
  CUtensorMap tmQ, tmK, tmV;
  FEMTO_TRY(make_tmap_2d_bf16(&tmQ, a.Q, (uint64_t)a.H * HD, N, a.q_stride, 64, BQ));
  FEMTO_TRY(make_tmap_2d_bf16(&tmK, a.K, (uint64_t)a.Hkv * HD, N, a.kv_stride, 64, BKV));
  FEMTO_TRY(make_tmap_2d_bf16(&tmV, a.V, (uint64_t)a.Hkv * HD, N, a.kv_stride, 64, BKV));
  FwdParams p;
  p.a = a;
  p.q_col0 = 0; p.k_col0 = 0; p.v_col0 = 0;
  static PerDevice attr;
  const int dev = PerDevice::current();
  if (dev < 0 || !attr.done[dev]) {
    CUDA_TRY(cudaFuncSetAttribute(attn_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM));
    CUDA_TRY(cudaFuncSetAttribute(attn_fwd_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM));
    CUDA_TRY(cudaFuncSetAttribute(attn_fwd_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PP_SMEM));
    if (dev >= 0) attr.done[dev] = true;
  }
  // FEMTO_ATTN_FWD in the environment selects an older kernel (measurement aid): 1 = one CTA per (query tile, head),
  // 3 = persistent, two query tiles in ping-pong (measured slower so far); default 2 = persistent, one query tile at a time
  static int variant = -1;
  if (variant < 0) { const char* e = getenv("FEMTO_ATTN_FWD"); variant = (e && e[0] >= '1' && e[0] <= '3') ? e[0] - '0' : 2; }
  // the persistent kernels assume every query tile is full and starts on a 16-byte boundary of the document starts
  if (variant == 3) {
    const int G = a.H / a.Hkv;
    const bool gqa = (G % 2) == 0;
    const int nqt = a.T / BQ;
    const int nitems = gqa ? nqt * (a.H / 2) * a.B : ((nqt + 1) / 2) * a.H * a.B;
    const int grid = std::min(nitems, device_sm_count());
    attn_fwd_pair_kernel<<<grid, FWD_THREADS, PP_SMEM, s>>>(tmQ, tmK, tmV, p, nitems, gqa ? 1 : 0, cycles_buffer());
    cycles_report("issuer: waiting / issuing", "softmax A, B: wait S / pass 1 / - / rescale / pass 2 / arrive / item end", 1, 1);
  } else if (variant == 2) {
    const int nitems = (a.T / BQ) * a.H * a.B;
    const int grid = std::min(nitems, device_sm_count());
    CUtensorMap tmO;   // O as [rows][H * 128] for 64-column x 32-row swizzled boxes (one per softmax warp)
    FEMTO_TRY(make_tmap_3d_bf16_sw(&tmO, a.O, (uint64_t)a.H * HD, N, 1, a.o_stride, 0, 64, 32, 3));
    attn_fwd_persistent_kernel<<<grid, FWD_THREADS, PF_SMEM, s>>>(tmQ, tmK, tmV, tmO, p, nitems, cycles_buffer());
    cycles_report("S issuer, P V issuer: waiting / issuing", "softmax (keys 0-63, 64-127): wait S / load+max / barrier / rescale / exp / arrive / item end", 1, 2);
  } else {
    dim3 grid(a.T / BQ, a.H, a.B);
    attn_fwd_tc_kernel<<<grid, FWD_THREADS, FWD_SMEM, s>>>(tmQ, tmK, tmV, p);
  }
  KERNEL_CHECK();
  return 0;
}

