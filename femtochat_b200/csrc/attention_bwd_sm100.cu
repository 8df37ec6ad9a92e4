// Reverse pass of flash attention (head_dim 128, bf16) on the sm_100a tensor cores, after
// src/kernels.jl:287-379 (P from the saved row statistics, dV += P^T dO, dP = dO V^T,
// dS = P o (dP - D), dQ += tau dS K, dK += tau dS^T Q).  The reference accumulates dQ with fp32
// atomics (ext/FemtoChatCUDAExt.jl:2002-2004); here two kernels each own their outputs, so every
// gradient is summed in a fixed order:
//   * dQ kernel: one CTA per 128 queries of a head; S = Q K^T and dP = dO V^T go to TMEM, the
//     row-owning threads (two per row, each half of the keys) turn them into dS (bf16, written
//     over S in TMEM), dQ += dS K stays in TMEM.
//   * dK/dV kernel: one CTA per 128 keys of a kv head; loops over the heads of the GQA group and
//     the query tiles that see these keys; S^T = K Q^T and dP^T = V dO^T go to TMEM, threads own
//     key rows and write P^T and dS^T back to TMEM, dV += P^T dO and dK += dS^T Q stay in TMEM.
#include <algorithm>

#include "sm100_ptx.cuh"

using namespace sm100;

namespace {

constexpr int HD = 128, BT = 128;
constexpr int TILE_BYTES = BT * HD * 2;  // two [128][64] swizzled slabs
constexpr int BWD_SMEM = TILE_BYTES * 6 + 1024 + 256 + 2 * 3 * 128 * 4;
constexpr float LOG2E = 1.4426950408889634f;

struct BwdParams {
  AttnArgs a;
  const float* D;   // [B][H][T] rowsum(dO*O)
  const float* L2;  // [B][H][T] lse * log2(e)
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
// Eight results leave as one 16-byte store; with `accumulate` the eight bf16 values already there are added first
// (Δattention!'s accumulate=true, ext/FemtoChatCUDAExt.jl:1775).
__device__ __forceinline__ void store8(bf16* dst, const uint32_t* r, float scale, bool accumulate) {
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; e++) v[e] = __uint_as_float(r[e]) * scale;
  if (accumulate) {
    const uint4 old = *reinterpret_cast<const uint4*>(dst);
    const bf16* oh = reinterpret_cast<const bf16*>(&old);
#pragma unroll
    for (int e = 0; e < 8; e++) v[e] += __bfloat162float(oh[e]);
  }
  uint4 q;
  uint32_t* w = reinterpret_cast<uint32_t*>(&q);
#pragma unroll
  for (int e = 0; e < 4; e++) w[e] = pack2(v[2 * e], v[2 * e + 1]);
  *reinterpret_cast<uint4*>(dst) = q;
}

// D[b][h][t] = sum_d dO*O and L2 = lse * log2(e): 16 lanes per (token, head) slice of 128 channels, 16-byte loads.
__global__ void __launch_bounds__(256) attn_bwd_prep_kernel(AttnArgs a, float* D, float* L2) {
  const long long total = (long long)a.B * a.T * a.H;
  const long long w0 = (long long)blockIdx.x * 16 + (threadIdx.x >> 4);
  const long long w = w0 < total ? w0 : total - 1;   // surplus half-warps recompute the last slice
  const int sub = threadIdx.x & 15;
  const int h = (int)(w % a.H);
  const long long row = w / a.H;
  const bf16* o = reinterpret_cast<const bf16*>(a.O) + row * a.o_stride + (long long)h * HD + sub * 8;
  const bf16* g = reinterpret_cast<const bf16*>(a.dO) + row * a.do_stride + (long long)h * HD + sub * 8;
  const uint4 ov = *reinterpret_cast<const uint4*>(o), gv = *reinterpret_cast<const uint4*>(g);
  const bf16* oh = reinterpret_cast<const bf16*>(&ov);
  const bf16* gh = reinterpret_cast<const bf16*>(&gv);
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) acc += __bfloat162float(oh[i]) * __bfloat162float(gh[i]);
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  const int b = (int)(row / a.T), t = (int)(row % a.T);
  if (sub == 0 && w0 < total) {
    const long long si = ((long long)b * a.H + h) * a.T + t;
    D[si] = acc;
    L2[si] = a.lse[si] * LOG2E;   // the exponent's offset in base 2, so P = exp2(S c - L2) is one FMA + ex2
  }
}

// A warp's 32 rows x 64 columns of a result (two tcgen05.ld chunks per thread, scaled) as bf16 into a 4 KB staging
// area in the 128-byte-swizzled layout of a (64 columns x 32 rows) TMA box: one tiled store then writes whole
// 128-byte lines, where sixteen-byte stores of one row per lane cost every store instruction 32 separate lines.
__device__ __forceinline__ void stage_rows(uint8_t* stage, const uint32_t (&r0)[32], const uint32_t (&r1)[32], float scale, int lane) {
#pragma unroll
  for (int u = 0; u < 2; u++) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
      uint4 q;
      uint32_t* w = reinterpret_cast<uint32_t*>(&q);
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const uint32_t a0 = u ? r1[8 * j + 2 * e] : r0[8 * j + 2 * e], a1 = u ? r1[8 * j + 2 * e + 1] : r0[8 * j + 2 * e + 1];
        w[e] = pack2(__uint_as_float(a0) * scale, __uint_as_float(a1) * scale);
      }
      *reinterpret_cast<uint4*>(stage + lane * 128 + (((u * 4 + j) ^ (lane & 7)) << 4)) = q;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// dQ kernel.  Roles: warp 0 streams K (three stages: a K tile is held until dQ has used it) and V
// (two stages) with TMA; warps 1, 3 and 2 issue dP = dO V^T, S = Q K^T and dQ += dS K (issue of
// tcgen05.mma blocks while the pipe is busy, so one issuer per product keeps it fed while another
// waits on a barrier); warps 4-11 own the query rows.  S is double-buffered in TMEM; dP has one buffer,
// which the threads release as soon as they hold its values in registers, so dP of the next tile
// is computed while they work on the current one.
// ------------------------------------------------------------------------------------------------
constexpr int DQ_SMEM = TILE_BYTES * 7 + 1024 + 256;

__global__ void __launch_bounds__(384, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmdQ, const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sdO = smem + TILE_BYTES;
  uint8_t* sK = smem + 2 * TILE_BYTES;  // 3 stages
  uint8_t* sV = smem + 5 * TILE_BYTES;  // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 7 * TILE_BYTES);
  uint64_t* qdo_full = bars;
  uint64_t* k_full = bars + 1;     // [3]
  uint64_t* k_free = bars + 4;     // [3] dQ of the tile in this stage has been executed
  uint64_t* v_full = bars + 7;     // [2]
  uint64_t* s_full = bars + 9;     // [2]
  uint64_t* dp_full = bars + 11;   // [2] indexed by tile parity (one TMEM buffer); also frees the tile's V stage
  uint64_t* dp_free = bars + 13;   // [1] every thread holds its part of dP in registers
  uint64_t* ds_ready = bars + 14;  // [2]
  uint64_t* dq_done = bars + 16;   // [2] dQ of a tile has been executed: its S/dS buffer may be overwritten
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const AttnArgs& a = p.a;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (a.H / a.Hkv);
  const int q0 = qt * BT;
  const int jhi = min(q0 + BT - 1, a.T - 1) / BT;
  int jlo = max(0, q0 - a.window_left) / BT;
  const long long row0 = (long long)b * a.T;
  if (a.doc_start) {
    // key tiles that lie before the earliest document start of these 128 queries are fully masked
    __shared__ int s_ds_min[4];
    if (threadIdx.x < 128) {
      const int v = __reduce_min_sync(0xffffffffu, a.doc_start[row0 + q0 + threadIdx.x]);
      if ((threadIdx.x & 31) == 0) s_ds_min[threadIdx.x >> 5] = v;
    }
    __syncthreads();
    jlo = max(jlo, min(min(s_ds_min[0], s_ds_min[1]), min(s_ds_min[2], s_ds_min[3])) / BT);
  }
  const int ntile = jhi - jlo + 1;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int i = 0; i < 3; i++) { mbar_init(&k_full[i], 1); mbar_init(&k_free[i], 1); }
    for (int i = 0; i < 2; i++) {
      mbar_init(&v_full[i], 1); mbar_init(&s_full[i], 1); mbar_init(&dp_full[i], 1);
      mbar_init(&ds_ready[i], 8); mbar_init(&dq_done[i], 1);
    }
    mbar_init(dp_free, 8);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS[2] = {tmem_base, tmem_base + 128};
  const uint32_t tdP = tmem_base + 256, tdQ = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(qdo_full, 2 * TILE_BYTES);
      tma_load_2d(sQ, &tmQ, qdo_full, h * HD, (int)(row0 + q0));
      tma_load_2d(sQ + TILE_BYTES / 2, &tmQ, qdo_full, h * HD + 64, (int)(row0 + q0));
      tma_load_2d(sdO, &tmdO, qdo_full, h * HD, (int)(row0 + q0));
      tma_load_2d(sdO + TILE_BYTES / 2, &tmdO, qdo_full, h * HD + 64, (int)(row0 + q0));
      for (int i = 0; i < ntile; i++) {
        const int ks = i % 3, vs = i & 1;
        const int krow = (int)(row0 + (jlo + i) * BT);
        if (i >= 3 && !mbar_wait(&k_free[ks], ((i - 3) / 3) & 1, abort_flag, a.status)) break;
        mbar_expect_tx(&k_full[ks], TILE_BYTES);
        tma_load_2d(sK + ks * TILE_BYTES, &tmK, &k_full[ks], kvh * HD, krow);
        tma_load_2d(sK + ks * TILE_BYTES + TILE_BYTES / 2, &tmK, &k_full[ks], kvh * HD + 64, krow);
        // the V stage of tile i-2 is free once its dP has been executed
        if (i >= 2 && !mbar_wait(&dp_full[vs], ((i - 2) >> 1) & 1, abort_flag, a.status)) break;
        mbar_expect_tx(&v_full[vs], TILE_BYTES);
        tma_load_2d(sV + vs * TILE_BYTES, &tmV, &v_full[vs], kvh * HD, krow);
        tma_load_2d(sV + vs * TILE_BYTES + TILE_BYTES / 2, &tmV, &v_full[vs], kvh * HD + 64, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- dP = dO V^T ----------------
      constexpr uint32_t idesc_kk = idesc_bf16(BT, BT, false, false);  // both operands K-major
      const uint32_t do_addr = smem_u32(sdO);
      bool ok = mbar_wait(qdo_full, 0, abort_flag, a.status);
      for (int i = 0; i < ntile && ok; i++) {
        const int st = i & 1;
        if (!mbar_wait(&v_full[st], (i >> 1) & 1, abort_flag, a.status)) break;
        // the single dP buffer is released early in the threads' work on tile i-1
        if (i >= 1 && !mbar_wait(dp_free, (i - 1) & 1, abort_flag, a.status)) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + st * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; k++) {
          const uint32_t off = (k >> 2) * (TILE_BYTES / 2) + (k & 3) * 32;
          mma_ss(tdP, smem_desc_sw128(do_addr + off, 16, 1024), smem_desc_sw128(v_addr + off, 16, 1024), idesc_kk, k > 0);
        }
        tc_commit(&dp_full[st]);
      }
    }
  } else if (warp == 3) {
    if (lane == 0) {
      // ---------------- S = Q K^T ----------------
      constexpr uint32_t idesc_kk = idesc_bf16(BT, BT, false, false);
      const uint32_t q_addr = smem_u32(sQ);
      bool ok = mbar_wait(qdo_full, 0, abort_flag, a.status);
      for (int i = 0; i < ntile && ok; i++) {
        const int st = i & 1, ks = i % 3;
        if (!mbar_wait(&k_full[ks], (i / 3) & 1, abort_flag, a.status)) break;
        // S(i) overwrites the buffer that held dS(i-2)
        if (i >= 2 && !mbar_wait(&dq_done[st], ((i - 2) >> 1) & 1, abort_flag, a.status)) break;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + ks * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; k++) {
          const uint32_t off = (k >> 2) * (TILE_BYTES / 2) + (k & 3) * 32;
          mma_ss(tS[st], smem_desc_sw128(q_addr + off, 16, 1024), smem_desc_sw128(k_addr + off, 16, 1024), idesc_kk, k > 0);
        }
        tc_commit(&s_full[st]);
      }
    }
  } else if (warp == 2) {
    if (lane == 0) {
      // ---------------- dQ += dS K ----------------
      constexpr uint32_t idesc_mn = idesc_bf16(BT, HD, false, true);   // A from TMEM, B N-contiguous
      for (int i = 0; i < ntile; i++) {
        const int st = i & 1, ks = i % 3;
        if (!mbar_wait(&ds_ready[st], (i >> 1) & 1, abort_flag, a.status)) break;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + ks * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < BT / 16; k++)  // 16 keys = 8 TMEM columns / 2048 B of K rows; dS of keys 64.. starts at column 64
          mma_ts(tdQ, tS[st] + (k >> 2) * 64 + (k & 3) * 8, smem_desc_sw128(k_addr + k * 2048, TILE_BYTES / 2, 1024), idesc_mn, (i > 0 || k > 0) ? 1u : 0u);
        tc_commit(&dq_done[st]);
        tc_commit(&k_free[ks]);
      }
    }
  } else if (warp >= 4) {
    const int quad = warp & 3;
    const int halfsel = (warp - 4) >> 2;  // warps 4-7 take key chunks 0,1 of each tile, warps 8-11 chunks 2,3
    const int r = quad * 32 + lane;
    const int q = q0 + r;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const float scale = rsqrtf((float)HD);
    const float c = scale * LOG2E;
    int lo = max(0, q - a.window_left);
    if (a.doc_start) lo = max(lo, a.doc_start[row0 + q]);
    const long long si = ((long long)b * a.H + h) * a.T + q;
    const float lse2 = p.L2[si];
    const float Dq = p.D[si];
    bool ok = true;
    for (int i = 0; i < ntile; i++) {
      const int st = i & 1;
      const int k0 = (jlo + i) * BT;
      if (ok && !mbar_wait(&dp_full[st], (i >> 1) & 1, abort_flag, a.status)) ok = false;
      if (ok && !mbar_wait(&s_full[st], (i >> 1) & 1, abort_flag, a.status)) ok = false;
      if (!ok) continue;
      tc_fence_after();
      const bool any_mask = __any_sync(0xffffffffu, (k0 + BT - 1 > q) || (k0 < lo));
      // The two threads of a row each take two 32-key chunks.  Both chunks of dP are read first and the
      // buffer is handed back, so the tensor core can fill it for the next tile meanwhile.  Each thread
      // writes its dS (bf16, 32 columns) over the start of its own 64 columns of S, once it has read them,
      // so the two threads of a row never touch each other's columns.
      uint32_t dr[2][32];
      tmem_ld32(tdP + lane_off + (2 * halfsel) * 32, dr[0]);
      tmem_ld32(tdP + lane_off + (2 * halfsel + 1) * 32, dr[1]);
      uint32_t pk[2][16];
#pragma unroll
      for (int u = 0; u < 2; u++) {
        const int cc = 2 * halfsel + u;
        uint32_t sr[32];
        tmem_ld32(tS[st] + lane_off + cc * 32, sr);
        tmem_ld_wait();
        if (u == 0) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(dp_free);
        }
        if (any_mask) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float d2[2];
#pragma unroll
            for (int e = 0; e < 2; e++) {
              const int k = k0 + cc * 32 + j + e;
              float pv = fast_exp2(__uint_as_float(sr[j + e]) * c - lse2);
              if (!(k <= q && k >= lo)) pv = 0.f;
              d2[e] = pv * (__uint_as_float(dr[u][j + e]) - Dq);
            }
            pk[u][j >> 1] = pack2(d2[0], d2[1]);
          }
        } else {   // no mask edge crosses this warp's rows in this tile: the common case, without the compares
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float p0 = fast_exp2(__uint_as_float(sr[j]) * c - lse2), p1 = fast_exp2(__uint_as_float(sr[j + 1]) * c - lse2);
            pk[u][j >> 1] = pack2(p0 * (__uint_as_float(dr[u][j]) - Dq), p1 * (__uint_as_float(dr[u][j + 1]) - Dq));
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 2; u++) tmem_st16(tS[st] + lane_off + halfsel * 64 + u * 16, pk[u]);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_ready[st]);
    }
    const int last = ntile - 1;
    if (ok && mbar_wait(&dq_done[last & 1], (last >> 1) & 1, abort_flag, a.status)) {
      tc_fence_after();
      if (!a.accumulate) {
        // every product has been executed: the Q tile's shared memory is free and stages the result for a TMA store
        uint32_t r0[32], r1[32];
        tmem_ld32(tdQ + lane_off + (2 * halfsel) * 32, r0);
        tmem_ld32(tdQ + lane_off + (2 * halfsel + 1) * 32, r1);
        tmem_ld_wait();
        uint8_t* stage = sQ + (warp - 4) * 4096;
        stage_rows(stage, r0, r1, scale, lane);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(&tmdQ, stage, h * HD + halfsel * 64, (int)(row0 + q0 + quad * 32), 0);
          bulk_commit();
          bulk_wait_read<0>();   // shared memory is released when the CTA leaves
        }
      } else {
        bf16* dq = reinterpret_cast<bf16*>(a.dQ) + (row0 + q) * a.dq_stride + (long long)h * HD;
#pragma unroll
        for (int cc = 2 * halfsel; cc < 2 * halfsel + 2; cc++) {
          uint32_t rr[32];
          tmem_ld32(tdQ + lane_off + cc * 32, rr);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 8) store8(dq + cc * 32 + j, rr + j, scale, true);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ------------------------------------------------------------------------------------------------
// dK / dV kernel.  A query tile is processed as two halves of 64 queries so that the S^T / dP^T
// buffers in TMEM (64 columns each) can be double-buffered next to the two 128-column accumulators:
// the tensor core computes the inputs of half h+1 and the dV / dK update of half h-1 while the
// threads turn half h into P^T and dS^T.  Warps 1 and 3 issue S^T = K Q^T and dP^T = V dO^T, warp 2
// issues dV += P^T dO and dK += dS^T Q (one issuer per product: tcgen05.mma issue blocks while the
// pipe is busy, so the barrier waits of one issuer overlap the issue of another).
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(384, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV,
                    const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE_BYTES;
  uint8_t* sQ = smem + 2 * TILE_BYTES;   // 2 stages
  uint8_t* sdO = smem + 4 * TILE_BYTES;  // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * TILE_BYTES);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;   // [2]
  uint64_t* qdo_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 5;     // [2] S^T of a half is in TMEM
  uint64_t* dp_full = bars + 7;    // [2] dP^T of a half is in TMEM
  uint64_t* pds_ready = bars + 9;  // [2] P^T and dS^T of a half are written
  uint64_t* out_done = bars + 11;  // [2] dV / dK of a half have been accumulated: its buffers may be overwritten
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stats = reinterpret_cast<float*>(smem + 6 * TILE_BYTES + 256);  // [2 stages][3][128]: lse * log2(e), D and document start of the tile's queries

  const AttnArgs& a = p.a;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int g = a.H / a.Hkv;
  const int k0 = kt * BT;
  const int ilo = kt;
  const int ihi = (int)min((long long)a.T / BT - 1, ((long long)k0 + BT - 1 + a.window_left) / BT);
  const long long row0 = (long long)b * a.T;
  // query tiles whose earliest document start lies after this key tile are fully masked: keep a
  // compact list of the visible ones (document starts need not be monotone for arbitrary positions)
  __shared__ int s_qlist[64];
  __shared__ int s_tmin[64];
  __shared__ int s_dsmax[64][4];   // per candidate tile: largest document start of each 32 queries
  __shared__ int s_nq;
  {
    const int cand = ihi - ilo + 1;
    if (a.doc_start) {
      for (int c = threadIdx.x >> 5; c < cand; c += 12) {
        const int base = (ilo + c) * BT + (threadIdx.x & 31) * 4;
        const int4 v = *reinterpret_cast<const int4*>(a.doc_start + row0 + base);
        const int m = __reduce_min_sync(0xffffffffu, min(min(v.x, v.y), min(v.z, v.w)));
        int mx = max(max(v.x, v.y), max(v.z, v.w));   // 8 lanes hold 32 consecutive queries
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        if ((threadIdx.x & 31) == 0) s_tmin[c] = m;
        if ((threadIdx.x & 7) == 0) s_dsmax[c][(threadIdx.x & 31) >> 3] = mx;
      }
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      int n = 0;
      for (int c = 0; c < cand; c++)
        if (!a.doc_start || s_tmin[c] <= k0 + BT - 1) s_qlist[n++] = ilo + c;
      s_nq = n;
    }
    __syncthreads();
  }
  const int nq = s_nq;         // >= 1: the diagonal tile always sees its own keys
  const int nit = nq * g;      // (head, query tile) pairs
  const int n2 = nit * 2;      // halves

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; i++) {
      mbar_init(&qdo_full[i], 1); mbar_init(&qdo_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&dp_full[i], 1); mbar_init(&pds_ready[i], 8); mbar_init(&out_done[i], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS[2] = {tmem_base, tmem_base + 64};
  const uint32_t tdP[2] = {tmem_base + 128, tmem_base + 192};
  const uint32_t tdK = tmem_base + 256, tdV = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * TILE_BYTES);
      tma_load_2d(sK, &tmK, kv_full, kvh * HD, (int)(row0 + k0));
      tma_load_2d(sK + TILE_BYTES / 2, &tmK, kv_full, kvh * HD + 64, (int)(row0 + k0));
      tma_load_2d(sV, &tmV, kv_full, kvh * HD, (int)(row0 + k0));
      tma_load_2d(sV + TILE_BYTES / 2, &tmV, kv_full, kvh * HD + 64, (int)(row0 + k0));
      for (int it = 0; it < nit; it++) {
        const int st = it & 1;
        const int h = kvh * g + it / nq;
        const int qrow = (int)(row0 + s_qlist[it % nq] * BT);
        if (!mbar_wait(&qdo_empty[st], ((it >> 1) & 1) ^ 1, abort_flag, a.status)) break;
        mbar_expect_tx(&qdo_full[st], 2 * TILE_BYTES + 1024 + (a.doc_start ? 512 : 0));
        const long long srow = ((long long)b * a.H + h) * a.T + s_qlist[it % nq] * BT;
        bulk_load_1d(stats + st * 384, p.L2 + srow, 512, &qdo_full[st]);
        bulk_load_1d(stats + st * 384 + 128, p.D + srow, 512, &qdo_full[st]);
        if (a.doc_start) bulk_load_1d(stats + st * 384 + 256, a.doc_start + qrow, 512, &qdo_full[st]);
        tma_load_2d(sQ + st * TILE_BYTES, &tmQ, &qdo_full[st], h * HD, qrow);
        tma_load_2d(sQ + st * TILE_BYTES + TILE_BYTES / 2, &tmQ, &qdo_full[st], h * HD + 64, qrow);
        tma_load_2d(sdO + st * TILE_BYTES, &tmdO, &qdo_full[st], h * HD, qrow);
        tma_load_2d(sdO + st * TILE_BYTES + TILE_BYTES / 2, &tmdO, &qdo_full[st], h * HD + 64, qrow);
      }
    }
  } else if (warp == 1 || warp == 3) {
    if (lane == 0) {
      // ---------------- S^T = K Q^T (warp 1) / dP^T = V dO^T (warp 3), 64 queries at a time ----------------
      constexpr uint32_t idesc_in = idesc_bf16(BT, 64, false, false);   // [128 keys] x [64 queries], K = head_dim
      const bool is_s = warp == 1;
      const uint32_t a_addr = smem_u32(is_s ? sK : sV);
      bool ok = mbar_wait(kv_full, 0, abort_flag, a.status);
      for (int h2 = 0; h2 < n2 && ok; h2++) {
        const int it = h2 >> 1, hf = h2 & 1, st = it & 1, bf = h2 & 1;
        if (hf == 0 && !mbar_wait(&qdo_full[st], (it >> 1) & 1, abort_flag, a.status)) break;
        // the buffer still holds P^T / dS^T of half h2-2 until its dV / dK update has been executed
        if (h2 >= 2 && !mbar_wait(&out_done[bf], ((h2 - 2) >> 1) & 1, abort_flag, a.status)) break;
        tc_fence_after();
        const uint32_t b_addr = smem_u32((is_s ? sQ : sdO) + st * TILE_BYTES) + hf * 8192;
        const uint32_t d_tmem = is_s ? tS[bf] : tdP[bf];
#pragma unroll
        for (int k = 0; k < HD / 16; k++) {
          const uint32_t off = (k >> 2) * (TILE_BYTES / 2) + (k & 3) * 32;
          mma_ss(d_tmem, smem_desc_sw128(a_addr + off, 16, 1024), smem_desc_sw128(b_addr + off, 16, 1024), idesc_in, k > 0);
        }
        tc_commit(is_s ? &s_full[bf] : &dp_full[bf]);
      }
    }
  } else if (warp == 2) {
    if (lane == 0) {
      // ---------------- dV += P^T dO, dK += dS^T Q over 64 queries ----------------
      constexpr uint32_t idesc_out = idesc_bf16(BT, HD, false, true);   // A from TMEM, B N-contiguous, K = 64 queries
      for (int h2 = 0; h2 < n2; h2++) {
        const int it = h2 >> 1, hf = h2 & 1, st = it & 1, bf = h2 & 1;
        if (!mbar_wait(&pds_ready[bf], (h2 >> 1) & 1, abort_flag, a.status)) break;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ + st * TILE_BYTES) + hf * 8192, do_addr = smem_u32(sdO + st * TILE_BYTES) + hf * 8192;
#pragma unroll
        for (int k = 0; k < 4; k++)
          mma_ts(tdV, tS[bf] + (k >> 1) * 32 + (k & 1) * 8, smem_desc_sw128(do_addr + k * 2048, TILE_BYTES / 2, 1024), idesc_out, (h2 > 0 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; k++)
          mma_ts(tdK, tdP[bf] + (k >> 1) * 32 + (k & 1) * 8, smem_desc_sw128(q_addr + k * 2048, TILE_BYTES / 2, 1024), idesc_out, (h2 > 0 || k > 0) ? 1u : 0u);
        tc_commit(&out_done[bf]);
        if (hf == 1) tc_commit(&qdo_empty[st]);
      }
    }
  } else if (warp >= 4) {
    const int quad = warp & 3;
    const int halfsel = (warp - 4) >> 2;  // which 32 of the 64 queries of a half this thread handles
    const int r = quad * 32 + lane;
    const int key = k0 + r;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const float scale = rsqrtf((float)HD);
    const float c = scale * LOG2E;
    bool ok = true;
    for (int h2 = 0; h2 < n2; h2++) {
      const int it = h2 >> 1, hf = h2 & 1, bf = h2 & 1;
      const int qi0 = s_qlist[it % nq] * BT + hf * 64;
      const float* sl = stats + (it & 1) * 384;
      const int qtile = s_qlist[it % nq];
      // the tile's statistics rows arrive with its Q / dO (already complete here: S^T was computed from them)
      if (ok && hf == 0 && !mbar_wait(&qdo_full[it & 1], (it >> 1) & 1, abort_flag, a.status)) ok = false;
      if (ok && !mbar_wait(&s_full[bf], (h2 >> 1) & 1, abort_flag, a.status)) ok = false;
      if (ok && !mbar_wait(&dp_full[bf], (h2 >> 1) & 1, abort_flag, a.status)) ok = false;
      if (!ok) continue;
      tc_fence_after();
      uint32_t pp[16], pd[16];
      {
        const int cq = hf * 64 + halfsel * 32;   // first query (within the tile) of this thread's chunk
        const int qf = qi0 + halfsel * 32;       // its position in the sequence
        uint32_t sr[32], dr[32];
        tmem_ld32(tS[bf] + lane_off + halfsel * 32, sr);
        tmem_ld32(tdP[bf] + lane_off + halfsel * 32, dr);
        // the mask matters only when some key of this warp is above the chunk's first query (causal edge)
        // or below the largest lower bound of its 32 queries (window / document edge)
        const int lo_max = max(max(0, qf + 31 - a.window_left), a.doc_start ? s_dsmax[qtile - ilo][cq >> 5] : 0);
        const bool need_mask = __any_sync(0xffffffffu, key > qf || key < lo_max);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 l4 = *reinterpret_cast<const float4*>(sl + cq + j);
            const float4 d4 = *reinterpret_cast<const float4*>(sl + 128 + cq + j);
            const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, dd[4] = {d4.x, d4.y, d4.z, d4.w};
            int los[4] = {0, 0, 0, 0};
            if (a.doc_start) {
              const int4 lo4 = *reinterpret_cast<const int4*>(sl + 256 + cq + j);
              los[0] = lo4.x; los[1] = lo4.y; los[2] = lo4.z; los[3] = lo4.w;
            }
            float p4[4], s4[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
              const int q = qf + j + e;
              float pv = fast_exp2(__uint_as_float(sr[j + e]) * c - ls[e]);
              if (!(key <= q && key >= max(los[e], q - a.window_left))) pv = 0.f;
              p4[e] = pv;
              s4[e] = pv * (__uint_as_float(dr[j + e]) - dd[e]);
            }
            pp[j >> 1] = pack2(p4[0], p4[1]); pp[(j >> 1) + 1] = pack2(p4[2], p4[3]);
            pd[j >> 1] = pack2(s4[0], s4[1]); pd[(j >> 1) + 1] = pack2(s4[2], s4[3]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 l4 = *reinterpret_cast<const float4*>(sl + cq + j);
            const float4 d4 = *reinterpret_cast<const float4*>(sl + 128 + cq + j);
            const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, dd[4] = {d4.x, d4.y, d4.z, d4.w};
            float p4[4], s4[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
              p4[e] = fast_exp2(__uint_as_float(sr[j + e]) * c - ls[e]);
              s4[e] = p4[e] * (__uint_as_float(dr[j + e]) - dd[e]);
            }
            pp[j >> 1] = pack2(p4[0], p4[1]); pp[(j >> 1) + 1] = pack2(p4[2], p4[3]);
            pd[j >> 1] = pack2(s4[0], s4[1]); pd[(j >> 1) + 1] = pack2(s4[2], s4[3]);
          }
        }
      }
      // P^T / dS^T of this thread's 32 queries go over the start of its own 32 columns of S^T / dP^T
      tmem_st16(tS[bf] + lane_off + halfsel * 32, pp);
      tmem_st16(tdP[bf] + lane_off + halfsel * 32, pd);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_ready[bf]);
    }
    const int lasth = n2 - 1;   // the dV / dK issuer's last commit covers every earlier instruction
    if (ok && mbar_wait(&out_done[lasth & 1], (lasth >> 1) & 1, abort_flag, a.status)) {
      tc_fence_after();
      if (!a.accumulate) {
        // every product has been executed: the two Q stages are free and stage dK and dV for TMA stores
        const int out_row = (int)(row0 + key) - lane;   // first of this warp's 32 key rows
#pragma unroll
        for (int which = 0; which < 2; which++) {
          uint32_t r0[32], r1[32];
          const uint32_t src = (which ? tdV : tdK) + lane_off;
          tmem_ld32(src + (2 * halfsel) * 32, r0);
          tmem_ld32(src + (2 * halfsel + 1) * 32, r1);
          tmem_ld_wait();
          uint8_t* stage = sQ + which * TILE_BYTES + (warp - 4) * 4096;
          stage_rows(stage, r0, r1, which ? 1.f : scale, lane);
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(which ? &tmdV : &tmdK, stage, kvh * HD + halfsel * 64, out_row, 0);
            bulk_commit();
          }
        }
        if (lane == 0) bulk_wait_read<0>();   // shared memory is released when the CTA leaves
      } else {
        bf16* dk = reinterpret_cast<bf16*>(a.dK) + (row0 + key) * a.dkv_stride + (long long)kvh * HD;
        bf16* dv = reinterpret_cast<bf16*>(a.dV) + (row0 + key) * a.dkv_stride + (long long)kvh * HD;
#pragma unroll
        for (int cc = 2 * halfsel; cc < 2 * halfsel + 2; cc++) {
          uint32_t rk[32], rv[32];
          tmem_ld32(tdK + lane_off + cc * 32, rk);
          tmem_ld32(tdV + lane_off + cc * 32, rv);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            store8(dk + cc * 32 + j, rk + j, scale, true);
            store8(dv + cc * 32 + j, rv + j, 1.f, true);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

}  // namespace

size_t attention_bwd_tc_ws_bytes(int B, int T, int H, int) { return 2 * sizeof(float) * (size_t)B * H * T; }

int attention_bwd_tc(const AttnArgs& a, cudaStream_t s) {
  if (!attention_tc_supported(a)) return femto_fail(FEMTO_ERR_UNSUPPORTED, "attention_bwd_tc: unsupported shape");
  if ((a.do_stride & 7) || (a.dq_stride & 7) || (a.dkv_stride & 7) || !aligned16(a.dO) || !aligned16(a.dQ) ||
      !aligned16(a.dK) || !aligned16(a.dV))
    return femto_fail(FEMTO_ERR_ALIGN, "attention_bwd_tc: gradient buffers must be 16-byte aligned");
  const size_t need = attention_bwd_tc_ws_bytes(a.B, a.T, a.H, a.hd);
  if (!a.ws || a.ws_bytes < need) return femto_fail(FEMTO_ERR_ARG, "attention_bwd_tc: workspace too small");
  const long long N = (long long)a.B * a.T;
  BwdParams p;
  p.a = a;
  p.D = reinterpret_cast<const float*>(a.ws);
  p.L2 = p.D + (size_t)a.B * a.H * a.T;
  attn_bwd_prep_kernel<<<cdiv(N * a.H, 16), 256, 0, s>>>(a, reinterpret_cast<float*>(a.ws), reinterpret_cast<float*>(a.ws) + (size_t)a.B * a.H * a.T);
  KERNEL_CHECK();
  CUtensorMap tmQ, tmK, tmV, tmdO;
  FEMTO_TRY(make_tmap_2d_bf16(&tmQ, a.Q, (uint64_t)a.H * HD, N, a.q_stride, 64, BT));
  FEMTO_TRY(make_tmap_2d_bf16(&tmK, a.K, (uint64_t)a.Hkv * HD, N, a.kv_stride, 64, BT));
  FEMTO_TRY(make_tmap_2d_bf16(&tmV, a.V, (uint64_t)a.Hkv * HD, N, a.kv_stride, 64, BT));
  FEMTO_TRY(make_tmap_2d_bf16(&tmdO, a.dO, (uint64_t)a.H * HD, N, a.do_stride, 64, BT));
  static PerDevice attr;
  const int dev = PerDevice::current();
  if (dev < 0 || !attr.done[dev]) {
    CUDA_TRY(cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM));
    CUDA_TRY(cudaFuncSetAttribute(attn_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM));
    if (dev >= 0) attr.done[dev] = true;
  }
  dim3 gq(a.T / BT, a.H, a.B);
  // result maps: 64-column x 32-row swizzled boxes, one per row-owning warp
  CUtensorMap tmdQ, tmdK, tmdV;
  FEMTO_TRY(make_tmap_3d_bf16_sw(&tmdQ, a.dQ, (uint64_t)a.H * HD, N, 1, a.dq_stride, 0, 64, 32, 3));
  FEMTO_TRY(make_tmap_3d_bf16_sw(&tmdK, a.dK, (uint64_t)a.Hkv * HD, N, 1, a.dkv_stride, 0, 64, 32, 3));
  FEMTO_TRY(make_tmap_3d_bf16_sw(&tmdV, a.dV, (uint64_t)a.Hkv * HD, N, 1, a.dkv_stride, 0, 64, 32, 3));
  attn_bwd_dq_kernel<<<gq, 384, DQ_SMEM, s>>>(tmQ, tmK, tmV, tmdO, tmdQ, p);
  KERNEL_CHECK();
  dim3 gk(a.T / BT, a.Hkv, a.B);
  attn_bwd_dkv_kernel<<<gk, 384, BWD_SMEM, s>>>(tmQ, tmK, tmV, tmdO, tmdK, tmdV, p);
  KERNEL_CHECK();
  return 0;
}
