// bf16 GEMM with fp32 accumulation on the sm_100a tensor cores.
//
// One persistent CTA per SM walks a list of (tile, k-range) units.  Warp 0 issues TMA tiled loads
// (128-byte swizzle) into a 4-stage shared-memory ring, warp 1 issues tcgen05.mma (128x256x16 per
// instruction) into one of two 256-column TMEM accumulators, warps 2-9 drain the other accumulator
// with tcgen05.ld and run the epilogue, so the epilogue of unit i overlaps the main loop of unit
// i+1.  Operands may be K-contiguous or M/N-contiguous in memory (the D x T x B layout of the
// reference makes the weight of a forward Linear N-contiguous and both operands of a weight
// gradient M/N-contiguous); the difference is only in the tensor maps and the matrix descriptors.
// Replaces the library GEMMs behind `W*X` (src/gpt.jl:28), the Linear/MLP reverse rules
// (ext/FemtoChatEnzymeExt.jl:83-134) and batched_mul! (ext/FemtoChatCUDAExt.jl:121-125).
#include <stdlib.h>

#include <algorithm>
#include <vector>

#include "sm100_ptx.cuh"

using namespace sm100;

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int A_BYTES = BM * BK * 2;
constexpr int STORE_STAGE_BYTES = 8 * 4096;  // 8 epilogue warps x [32 rows][64 bf16]
constexpr int NTHREADS = 320;  // TMA warp, MMA warp, 8 epilogue warps (two per TMEM lane quadrant)
constexpr int TMEM_COLS = 512;
constexpr int MAX_STAGES = 6;

// One CTA per 128 x 256 tile (PAIR = false), or a pair of CTAs of one cluster per 256 x 256 tile (PAIR = true):
// tcgen05.mma.cta_group::2 multiplies 256 rows at once, each CTA holding 128 rows of A and HALF of B's columns in
// its own shared memory and its own 128 x 256 accumulator in its own TMEM.  A pair moves 2 x (16 + 16) KB of
// operands per k-block where two single CTAs move 2 x (16 + 32) KB: a third less shared-memory and L2 traffic per
// flop, and the smaller stages leave room for a six-deep ring.
template <bool PAIR> struct Geo {
  static constexpr int TILE_M = PAIR ? 2 * BM : BM;          // rows of an output tile (unit of scheduling)
  static constexpr int BN_LOCAL = PAIR ? BN / 2 : BN;        // columns of B this CTA loads
  static constexpr int B_BYTES = BN_LOCAL * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = PAIR ? 6 : 4;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STORE_STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int SLOTS = PAIR ? 2 : 1;                 // 128-row halves per unit (split-K partial slots)
};

struct TcParams {
  GemmArgs g;
  int tiles_m, tiles_n, kblocks, splits, kb_per_split, total_units;
  float* partial;  // [unit][8 chunks][128 rows][32 cols] when splits > 1
  int tma_store;   // bf16 results leave through shared memory and TMA tiled stores
  int pair;        // units are 256-row tiles computed by CTA pairs
  int a_slabs, b_slabs;  // an M/N-contiguous operand arrives with one 4-d copy per k-block instead of one per 64-wide slab
  int stages;      // depth of the operand ring (<= Geo::STAGES; fewer stages leave shared memory to co-resident kernels)
};

// Tile rasterisation: groups of GROUP_M row-tiles are walked column by column, so one wave of CTAs
// covers a roughly square patch of the output (16 x 9 tiles) and re-reads neither operand from HBM.
constexpr int GROUP_M = 16;
__device__ __forceinline__ void tile_coords(const TcParams& p, int t, int& bz, int& mt, int& nt) {
  const int per = p.tiles_m * p.tiles_n;
  bz = t / per;
  const int pid = t % per;
  const int width = GROUP_M * p.tiles_n;
  const int first_m = (pid / width) * GROUP_M;
  const int gsz = min(p.tiles_m - first_m, GROUP_M);
  mt = first_m + (pid % width) % gsz;
  nt = (pid % width) / gsz;
}

__device__ __forceinline__ float sqrt_approx(float x) {
  float y;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float softcap15(float x) {
  // 15 * tanh(x/15) on the special-function unit (tanh.approx: relative error about 2^-11, below the
  // bf16 rounding of the logits that feed it)
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x * (1.f / 15.f)));
  return 15.f * t;
}

__device__ __forceinline__ float* f32_dst(const GemmArgs& g, long long bz, int m, int n) {
  if (g.nseg == 0) return reinterpret_cast<float*>(g.C) + bz * g.strideC + (long long)m * g.ldc + n;
  for (int s = 0; s < g.nseg; s++)
    if (n >= g.seg_col0[s] && n < g.seg_col0[s] + g.seg_ncol[s])
      return g.seg_ptr[s] + (long long)m * g.seg_ld[s] + (n - g.seg_col0[s]);
  return nullptr;
}

// A warp's results leave in blocks of 32 rows x 64 columns (two adjacent 32-column chunks): each lane writes
// its row into shared memory (128-byte rows, 128-byte swizzle, so the 16-byte stores of eight lanes hit distinct
// banks) and one TMA tiled store writes whole 128-byte lines, clipping rows >= M and columns >= N.
// sub: 0 = first chunk of the pair (waits until the previous store has read the buffer), 1 = second;
// flush: this chunk is the last valid one of its pair.
__device__ __forceinline__ void stage_store_bf16(const float (&v)[32], uint8_t* stage_buf, const CUtensorMap* tmC, int sub, bool flush,
                                                 int nc_pair, int m_warp0, int bz, int lane) {
  if (sub == 0) {
    if (lane == 0) bulk_wait_read<0>();
    __syncwarp();
  }
#pragma unroll
  for (int j = 0; j < 4; j++) {
    uint4 q;
    __nv_bfloat162* hq = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
    for (int e = 0; e < 4; e++) hq[e] = __floats2bfloat162_rn(v[8 * j + 2 * e], v[8 * j + 2 * e + 1]);
    *reinterpret_cast<uint4*>(stage_buf + lane * 128 + (((sub * 4 + j) ^ (lane & 7)) << 4)) = q;
  }
  if (flush) {
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      tma_store_3d(tmC, stage_buf, nc_pair, m_warp0, bz);
      bulk_commit();
    }
  }
}

// Tiles of a symmetric result that no element of the upper triangle touches (every role skips the same units).
__device__ __forceinline__ bool below_diagonal(const GemmArgs& g, int mt, int nt, int tile_m) {
  return g.upper_only && (nt + 1) * BN <= mt * tile_m;
}

// One 32-column chunk of one output row with a bf16 result: C = f(acc, aux).
template <int EPI>
__device__ __forceinline__ void bf16_chunk(const GemmArgs& g, float (&v)[32], int bz, int m, int nc, bool full_chunk,
                                           const uint4 (&pre)[4], bool use_pre, bool row_ok,
                                           uint8_t* stage_buf, const CUtensorMap* tmC, int sub, bool flush, int nc_pair, int m_warp0,
                                           int lane) {
  bf16* C = reinterpret_cast<bf16*>(g.C) + (long long)bz * g.strideC + (long long)m * g.ldc + nc;
  constexpr bool need_aux = EPI == EPI_RESID || EPI == EPI_DRELU2 || EPI == EPI_AXPBY;
  const bool vec = full_chunk && (g.ldc & 7) == 0 && (!need_aux || (g.ldaux & 7) == 0);
  float a[32];
  if constexpr (need_aux) {
    const bf16* aux = reinterpret_cast<const bf16*>(g.aux) + (long long)bz * g.strideAux + (long long)m * g.ldaux + nc;
    if (!row_ok) {
#pragma unroll
      for (int j = 0; j < 32; j++) a[j] = 0.f;
    } else if (vec) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        // `pre` was loaded one chunk ahead (while the previous chunk was being processed)
        uint4 q = use_pre ? pre[j >> 3] : *reinterpret_cast<const uint4*>(aux + j);
        const bf16* hq = reinterpret_cast<const bf16*>(&q);
#pragma unroll
        for (int e = 0; e < 8; e++) a[j + e] = __bfloat162float(hq[e]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; j++) a[j] = (nc + j < g.N) ? __bfloat162float(aux[j]) : 0.f;
    }
  }
  const float alpha = g.alpha, beta = g.beta;
#pragma unroll
  for (int j = 0; j < 32; j++) {
    float x = v[j];
    if constexpr (EPI == EPI_RESID) x = a[j] + x;
    if constexpr (EPI == EPI_RELU2) { x = fmaxf(x, 0.f); x = x * x; }
    if constexpr (EPI == EPI_DRELU2) x = x * 2.f * sqrt_approx(fmaxf(a[j], 0.f));
    if constexpr (EPI == EPI_AXPBY) x = alpha * a[j] + beta * x;
    v[j] = x;
  }
  if (stage_buf != nullptr) {
    stage_store_bf16(v, stage_buf, tmC, sub, flush, nc_pair, m_warp0, bz, lane);
  } else if (!row_ok) {
    // nothing to store for rows past M
  } else if (vec) {
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      uint4 q;
      __nv_bfloat162* hq = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
      for (int e = 0; e < 4; e++) hq[e] = __floats2bfloat162_rn(v[j + 2 * e], v[j + 2 * e + 1]);
      *reinterpret_cast<uint4*>(C + j) = q;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; j++) if (nc + j < g.N) C[j] = __float2bfloat16_rn(v[j]);
  }
}

template <bool A_K, bool B_K, bool PAIR>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const TcParams p) {
  typedef Geo<PAIR> G;
  constexpr int STAGE_BYTES = G::STAGE_BYTES, TILE_M = G::TILE_M;
  const int STAGES = p.stages;
  extern __shared__ uint8_t smem_raw[];
  // the same offsets in both CTAs of a pair: the shared-memory window of every CTA starts on the same alignment
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* store_stage = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES + STORE_STAGE_BYTES);
  uint64_t* full = bars;                 // [STAGES]
  uint64_t* empty = bars + STAGES;       // [STAGES]
  uint64_t* tfull = bars + 2 * STAGES;   // [2]
  uint64_t* tempty = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const GemmArgs& g = p.g;
  // In a pair the even CTA (rank 0) is the leader: its thread issues the MMAs of both, its `full` barriers count
  // the bytes of both CTAs' loads and its `tempty` barriers the epilogue warps of both.
  const int rank = PAIR ? (int)cluster_ctarank() : 0;
  const int first_unit = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int unit_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; i++) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; i++) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], PAIR ? 16 : 8); }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (PAIR) {
    // the peer's barriers must exist before anything of this CTA can signal them
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    if (PAIR) { tmem_alloc2(tmem_slot, TMEM_COLS); tmem_relinquish2(); }
    else { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above touched no global memory: it may overlap the tail of the previous kernel in the stream.
  grid_launch_dependents();
  grid_dependency_wait();

  auto unit_coords = [&](int u, int& bz, int& mt, int& nt, int& kb0, int& kb1) {
    // split-major: all tiles of one k-range run together, so the 148 CTAs stream the same rows of
    // both operands through L2 at the same time
    const int ntile = p.tiles_m * p.tiles_n * p.g.batch;
    const int s = u / ntile;
    tile_coords(p, u % ntile, bz, mt, nt);
    kb0 = s * p.kb_per_split;
    kb1 = min(p.kblocks, kb0 + p.kb_per_split);
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      uint32_t issued_mask = 0, last_parity = 0;
      bool ok = true;
      for (int u = first_unit; u < p.total_units && ok; u += unit_step) {
        int bz, mt, nt, kb0, kb1;
        unit_coords(u, bz, mt, nt, kb0, kb1);
        if (below_diagonal(g, mt, nt, TILE_M)) continue;
        const int m0 = mt * TILE_M + rank * BM;           // first row of A this CTA loads
        const int n0 = nt * BN + rank * G::BN_LOCAL;      // first column of B this CTA loads (its half, in a pair)
        for (int kb = kb0; kb < kb1; kb++) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, g.status)) { ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          if (PAIR) {
            // the leader announces the bytes of both CTAs; the loads of either CTA are counted on its barrier
            if (rank == 0) mbar_expect_tx(&full[stage], 2 * STAGE_BYTES);
            if (A_K) tma_load_3d_pair(sa, &tmA, &full[stage], kb * BK, m0, bz);
            else tma_load_4d_pair(sa, &tmA, &full[stage], 0, kb * BK, m0 / 64, bz);
            if (B_K) tma_load_3d_pair(sb, &tmB, &full[stage], kb * BK, n0, bz);
            else tma_load_4d_pair(sb, &tmB, &full[stage], 0, kb * BK, n0 / 64, bz);
          } else {
          mbar_expect_tx(&full[stage], STAGE_BYTES);
          if (A_K) {
            tma_load_3d(sa, &tmA, &full[stage], kb * BK, mt * BM, bz);
          } else if (p.a_slabs) {
            tma_load_4d(sa, &tmA, &full[stage], 0, kb * BK, mt * (BM / 64), bz);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; j++) tma_load_3d(sa + j * 8192, &tmA, &full[stage], mt * BM + j * 64, kb * BK, bz);
          }
          if (B_K) {
            tma_load_3d(sb, &tmB, &full[stage], kb * BK, nt * BN, bz);
          } else if (p.b_slabs) {
            tma_load_4d(sb, &tmB, &full[stage], 0, kb * BK, nt * (BN / 64), bz);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; j++) tma_load_3d(sb + j * 8192, &tmB, &full[stage], nt * BN + j * 64, kb * BK, bz);
          }
          }
          issued_mask |= 1u << stage;
          last_parity = (last_parity & ~(1u << stage)) | (phase << stage);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (*abort_flag && !PAIR) {
        // let loads already in flight land before the CTA exits (a pair meets at the cluster barrier below, and
        // only the leader's barriers see the bytes)
        for (int i = 0; i < STAGES; i++)
          if (issued_mask & (1u << i))
            for (uint32_t it = 0; it < WAIT_LIMIT && !mbar_try_wait(&full[i], (last_parity >> i) & 1u); ++it) {}
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = idesc_bf16(TILE_M, BN, !A_K, !B_K);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int u = first_unit; u < p.total_units && ok; u += unit_step) {
        int bz, mt, nt, kb0, kb1;
        unit_coords(u, bz, mt, nt, kb0, kb1);
        if (below_diagonal(g, mt, nt, TILE_M)) continue;
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag, g.status)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; kb++) {
          if (!mbar_wait(&full[stage], phase, abort_flag, g.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; k++) {
            // K-major: rows of 128 B, 8-row groups 1024 B apart, 16 k-elements = 32 B along the row.
            // MN-major: [64 k][64 mn] slabs of 8192 B, 8-k groups 1024 B apart, 16 k = 2048 B.
            const uint64_t ad = A_K ? smem_desc_sw128(sa + k * 32, 16, 1024) : smem_desc_sw128(sa + k * 2048, 8192, 1024);
            const uint64_t bd = B_K ? smem_desc_sw128(sb + k * 32, 16, 1024) : smem_desc_sw128(sb + k * 2048, 8192, 1024);
            if (PAIR) mma_ss_pair(d_tmem, ad, bd, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            else mma_ss(d_tmem, ad, bd, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          if (PAIR) tc_commit_pair(&empty[stage]); else tc_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (PAIR) tc_commit_pair(&tfull[acc]); else tc_commit(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ---------------- epilogue (warps 2..9) ----------------
    const int quad = warp & 3;           // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;    // the two warps of a quadrant take alternate pairs of 32-column chunks
    const int row_in_tile = quad * 32 + lane;
    int acc = 0; uint32_t acc_phase = 0;
    for (int u = first_unit; u < p.total_units; u += unit_step) {
      int bz, mt, nt, kb0, kb1;
      unit_coords(u, bz, mt, nt, kb0, kb1);
      if (below_diagonal(g, mt, nt, TILE_M)) continue;
      if (!mbar_wait(&tfull[acc], acc_phase, abort_flag, g.status)) break;
      tc_fence_after();
      const int m_tile0 = mt * TILE_M + rank * BM;   // first row of this CTA's 128 x 256 part of the tile
      const int m = m_tile0 + row_in_tile;
      const int n0 = nt * BN;
      const bool row_ok = m < g.M;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quad * 32) << 16);
      // cross-entropy row state
      float rmax = -INFINITY, rsum = 0.f;
      int tgt = -1;
      if (g.epi == EPI_XENT_STATS && row_ok) tgt = g.targets0[m];
      // operands of the residual / relu^2-reverse / axpby epilogues are fetched one chunk ahead
      const bool aux_epi = p.splits == 1 && (g.epi == EPI_RESID || g.epi == EPI_DRELU2 || g.epi == EPI_AXPBY) &&
                           (g.ldaux & 7) == 0 && (g.ldc & 7) == 0 && row_ok;
      const bf16* aux_row = aux_epi ? reinterpret_cast<const bf16*>(g.aux) + (long long)bz * g.strideAux + (long long)m * g.ldaux : nullptr;
      uint4 auxq[4], auxn[4];
      // this warp's chunks in order: 2*half, 2*half+1, 4+2*half, 4+2*half+1 (64 adjacent columns leave in one store)
      auto chunk_of = [&](int ci) { return (ci >> 1) * 4 + 2 * half + (ci & 1); };
      bool pre_ok = false, next_ok = aux_epi && n0 + chunk_of(0) * 32 + 32 <= g.N;
      if (next_ok) {
#pragma unroll
        for (int j = 0; j < 4; j++) auxn[j] = *reinterpret_cast<const uint4*>(aux_row + n0 + chunk_of(0) * 32 + j * 8);
      }
#pragma unroll 1
      for (int ci = 0; ci < BN / 64; ci++) {
        const int c = chunk_of(ci);
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(taddr + c * 32, r);
        pre_ok = next_ok;
#pragma unroll
        for (int j = 0; j < 4; j++) auxq[j] = auxn[j];
        const int cn = chunk_of(ci + 1);
        next_ok = aux_epi && ci + 1 < BN / 64 && n0 + cn * 32 + 32 <= g.N;
        if (next_ok) {
#pragma unroll
          for (int j = 0; j < 4; j++) auxn[j] = *reinterpret_cast<const uint4*>(aux_row + n0 + cn * 32 + j * 8);
        }
        tmem_ld_wait();
        const int nc = n0 + c * 32;
        const bool tma_out = p.tma_store != 0 && p.splits == 1 && g.epi != EPI_F32;
        if (nc >= g.N || (!row_ok && !tma_out)) continue;   // on the TMA path the whole warp stays together
        uint8_t* sbuf = tma_out ? store_stage + (warp - 2) * 4096 : nullptr;
        const int sub = ci & 1, nc_pair = n0 + (c & ~1) * 32;
        const bool flush = sub == 1 || nc + 32 >= g.N;   // last valid chunk of its pair
        const bool full_chunk = nc + 32 <= g.N;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
        if (p.splits > 1) {
          float* dst = p.partial + (((long long)u * G::SLOTS + rank) * 8 + c) * (128 * 32) + row_in_tile * 32;
#pragma unroll
          for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          continue;
        }
        switch (g.epi) {
          case EPI_F32: {
            float* dst = reinterpret_cast<float*>(g.C) + (long long)bz * g.strideC + (long long)m * g.ldc + nc;
            if (g.nseg == 0 && full_chunk && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o = make_float4(g.alpha * v[j], g.alpha * v[j + 1], g.alpha * v[j + 2], g.alpha * v[j + 3]);
                if (g.beta != 0.f) {
                  float4 q = *reinterpret_cast<const float4*>(dst + j);
                  o.x += q.x; o.y += q.y; o.z += q.z; o.w += q.w;
                }
                *reinterpret_cast<float4*>(dst + j) = o;
              }
            } else if (g.nseg == 0 && full_chunk && (reinterpret_cast<uintptr_t>(dst) & 15) == 8) {
              // delta ranges start at even element offsets: an 8-byte aligned row is handled as 2 + 7 x 4 + 2 floats
              auto rmw2 = [&](int j) {
                float2 o = make_float2(g.alpha * v[j], g.alpha * v[j + 1]);
                if (g.beta != 0.f) { const float2 q = *reinterpret_cast<const float2*>(dst + j); o.x += q.x; o.y += q.y; }
                *reinterpret_cast<float2*>(dst + j) = o;
              };
              rmw2(0);
#pragma unroll
              for (int j = 2; j < 30; j += 4) {
                float4 o = make_float4(g.alpha * v[j], g.alpha * v[j + 1], g.alpha * v[j + 2], g.alpha * v[j + 3]);
                if (g.beta != 0.f) {
                  float4 q = *reinterpret_cast<const float4*>(dst + j);
                  o.x += q.x; o.y += q.y; o.z += q.z; o.w += q.w;
                }
                *reinterpret_cast<float4*>(dst + j) = o;
              }
              rmw2(30);
            } else {
#pragma unroll
              for (int j = 0; j < 32; j++) {
                if (nc + j < g.N) {
                  float* dst = f32_dst(g, bz, m, nc + j);
                  if (dst) *dst = (g.beta != 0.f ? *dst : 0.f) + g.alpha * v[j];
                }
              }
            }
          } break;
          case EPI_XENT_STATS: {
            // with a destination the raw logits are kept in bf16 (as the reference materialises them) and
            // the statistics are taken from the rounded values, so a later pass over the stored chunk agrees
            if (tma_out) {
#pragma unroll
              for (int j = 0; j < 32; j++) v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
              stage_store_bf16(v, sbuf, &tmC, sub, flush, nc_pair, m_tile0 + quad * 32, bz, lane);
            }
            float cm = -INFINITY;
#pragma unroll
            for (int j = 0; j < 32; j++) {
              v[j] = (nc + j < g.vocab) ? softcap15(v[j]) : -INFINITY;
              cm = fmaxf(cm, v[j]);
            }
            if (tgt >= nc && tgt < nc + 32) {
#pragma unroll
              for (int j = 0; j < 32; j++) if (nc + j == tgt) g.tz[m] = v[j];
            }
            const float nm = fmaxf(rmax, cm);
            float cs = 0.f;
#pragma unroll
            for (int j = 0; j < 32; j++) cs += __expf(v[j] - nm);
            rsum = rsum * __expf(rmax - nm) + cs;
            rmax = nm;
          } break;
          case EPI_STORE: bf16_chunk<EPI_STORE>(g, v, bz, m, nc, full_chunk, auxq, pre_ok, row_ok, sbuf, &tmC, sub, flush, nc_pair, m_tile0 + quad * 32, lane); break;
          case EPI_RESID: bf16_chunk<EPI_RESID>(g, v, bz, m, nc, full_chunk, auxq, pre_ok, row_ok, sbuf, &tmC, sub, flush, nc_pair, m_tile0 + quad * 32, lane); break;
          case EPI_RELU2: bf16_chunk<EPI_RELU2>(g, v, bz, m, nc, full_chunk, auxq, pre_ok, row_ok, sbuf, &tmC, sub, flush, nc_pair, m_tile0 + quad * 32, lane); break;
          case EPI_DRELU2: bf16_chunk<EPI_DRELU2>(g, v, bz, m, nc, full_chunk, auxq, pre_ok, row_ok, sbuf, &tmC, sub, flush, nc_pair, m_tile0 + quad * 32, lane); break;
          case EPI_AXPBY: bf16_chunk<EPI_AXPBY>(g, v, bz, m, nc, full_chunk, auxq, pre_ok, row_ok, sbuf, &tmC, sub, flush, nc_pair, m_tile0 + quad * 32, lane); break;
          default: break;
        }
      }
      if (g.epi == EPI_XENT_STATS && row_ok && p.splits == 1) g.stats[((long long)m * p.tiles_n + nt) * 2 + half] = make_float2(rmax, rsum);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { if (PAIR) mbar_arrive_even(&tempty[acc]); else mbar_arrive(&tempty[acc]); }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  if (warp >= 2 && lane == 0) bulk_wait_all();   // every TMA store of this warp has landed
  tc_fence_before();
  __syncthreads();
  if (PAIR) {
    // neither CTA may free the pair's tensor memory, or leave while the peer can still signal its barriers,
    // before both are done
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc2(tmem_base, TMEM_COLS); else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Sum the split-K partials in split order and apply the fp32 epilogue.  One block per
// (tile, 32-column chunk): 128 rows x 32 columns, one float4 column group per thread and row slice.
__global__ void __launch_bounds__(256) gemm_tc_reduce_kernel(const TcParams p) {
  const GemmArgs& g = p.g;
  // blockIdx.x enumerates (tile, 128-row half of it, 32-column chunk); a tile has two halves when CTA pairs made it
  const int slots = p.pair ? 2 : 1;
  const int c = blockIdx.x & 7, half_id = (blockIdx.x >> 3) % slots, tile = (blockIdx.x >> 3) / slots;
  const int ntile = p.tiles_m * p.tiles_n * g.batch;
  int bz, mt, nt;
  tile_coords(p, tile, bz, mt, nt);
  const int tile_m = p.pair ? 2 * BM : BM;
#pragma unroll
  for (int it = 0; it < 4; it++) {
    const int e = it * 256 + threadIdx.x;     // 0..1023 float4 groups of this chunk
    const int row = e >> 3, j4 = (e & 7) * 4;
    const int m = mt * tile_m + half_id * BM + row, n = nt * BN + c * 32 + j4;
    if (m >= g.M || n >= g.N) continue;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* src = p.partial + (((long long)tile * slots + half_id) * 8 + c) * (128 * 32) + row * 32 + j4;
    const long long sstride = (long long)ntile * slots * 8 * (128 * 32);
    for (int s = 0; s < p.splits; s++) {
      const float4 q = *reinterpret_cast<const float4*>(src + s * sstride);
      acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
    }
    // destination of the four columns: one range of delta, or one of the segments of a fused product (segment
    // boundaries are multiples of 4 in practice, checked here).  delta ranges start at even element offsets, so the
    // address is 16-byte aligned or 8-byte aligned; both get vector accesses.
    float* dst = g.nseg == 0 ? reinterpret_cast<float*>(g.C) + (long long)bz * g.strideC + (long long)m * g.ldc + n
                             : f32_dst(g, bz, m, n);
    const bool contiguous = dst != nullptr && n + 3 < g.N && (g.nseg == 0 || f32_dst(g, bz, m, n + 3) == dst + 3);
    const uintptr_t ph = reinterpret_cast<uintptr_t>(dst) & 15;
    float4 o = make_float4(g.alpha * acc.x, g.alpha * acc.y, g.alpha * acc.z, g.alpha * acc.w);
    if (contiguous && ph == 0) {
      if (g.beta != 0.f) {
        const float4 q = *reinterpret_cast<const float4*>(dst);
        o.x += q.x; o.y += q.y; o.z += q.z; o.w += q.w;
      }
      *reinterpret_cast<float4*>(dst) = o;
    } else if (contiguous && ph == 8) {
      if (g.beta != 0.f) {
        const float2 q0 = *reinterpret_cast<const float2*>(dst), q1 = *reinterpret_cast<const float2*>(dst + 2);
        o.x += q0.x; o.y += q0.y; o.z += q1.x; o.w += q1.y;
      }
      *reinterpret_cast<float2*>(dst) = make_float2(o.x, o.y);
      *reinterpret_cast<float2*>(dst + 2) = make_float2(o.z, o.w);
    } else {
      const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        if (n + j < g.N) {
          float* d1 = f32_dst(g, bz, m, n + j);
          if (d1) *d1 = (g.beta != 0.f ? *d1 : 0.f) + g.alpha * vals[j];
        }
      }
    }
  }
}

}  // namespace

// ---- host ---------------------------------------------------------------------------------------
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static PFN_encodeTiled get_encode() {
  static PFN_encodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess && p)
      fn = reinterpret_cast<PFN_encodeTiled>(p);
  }
  return fn;
}

int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t dim0, uint64_t dim1, uint64_t dim2,
                      uint64_t stride1_elems, uint64_t stride2_elems, uint32_t box0, uint32_t box1) {
  return make_tmap_3d_bf16_sw(out, base, dim0, dim1, dim2, stride1_elems, stride2_elems, box0, box1, 3);
}

int make_tmap_3d_bf16_sw(CUtensorMap* out, const void* base, uint64_t dim0, uint64_t dim1, uint64_t dim2,
                         uint64_t stride1_elems, uint64_t stride2_elems, uint32_t box0, uint32_t box1, int swizzle) {
  PFN_encodeTiled enc = get_encode();
  if (!enc) return femto_fail(FEMTO_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {dim0, dim1, dim2 ? dim2 : 1};
  cuuint64_t strides[2] = {stride1_elems * 2, (dim2 > 1 ? stride2_elems : stride1_elems * dim1) * 2};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapSwizzle sw = swizzle == 3 ? CU_TENSOR_MAP_SWIZZLE_128B : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                                : swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return femto_fail(FEMTO_ERR_ALIGN, "cuTensorMapEncodeTiled failed (%d): dims %llu x %llu x %llu, row stride %llu B",
                      (int)r, (unsigned long long)dim0, (unsigned long long)dim1, (unsigned long long)dims[2],
                      (unsigned long long)strides[0]);
  return 0;
}

int make_tmap_4d_slabs_bf16(CUtensorMap* out, const void* base, uint64_t extent, uint64_t K, uint64_t batch, uint64_t ld_elems,
                            uint64_t batch_stride_elems, uint32_t box_k, uint32_t slabs) {
  PFN_encodeTiled enc = get_encode();
  if (!enc || (extent & 63)) return 1;
  cuuint64_t dims[4] = {64, K, extent / 64, batch ? batch : 1};
  cuuint64_t strides[3] = {ld_elems * 2, 128, (batch > 1 ? batch_stride_elems : ld_elems * K) * 2};
  cuuint32_t box[4] = {64, box_k, slabs, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1;
}

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t dim0, uint64_t dim1, uint64_t stride1_elems,
                      uint32_t box0, uint32_t box1) {
  PFN_encodeTiled enc = get_encode();
  if (!enc) return femto_fail(FEMTO_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {dim0, dim1};
  cuuint64_t strides[1] = {stride1_elems * 2};
  cuuint32_t box[2] = {box0, box1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return femto_fail(FEMTO_ERR_ALIGN, "cuTensorMapEncodeTiled (2d) failed (%d): dims %llu x %llu, row stride %llu B", (int)r,
                      (unsigned long long)dim0, (unsigned long long)dim1, (unsigned long long)strides[0]);
  return 0;
}

bool gemm_tc_supported(const GemmArgs& g) {
  if (g.M < BM || g.N < BN || g.K < BK) return false;
  if ((g.lda & 7) || (g.ldb & 7) || (g.strideA & 7) || (g.strideB & 7)) return false;
  if (!aligned16(g.A) || !aligned16(g.B)) return false;
  // the contiguous extent of an M/N-major operand must cover whole 16-byte units
  if (!g.a_kmajor && (g.M & 7)) return false;
  if (!g.b_kmajor && (g.N & 7)) return false;
  if (g.a_kmajor && (g.K & 7)) return false;
  if (g.b_kmajor && (g.K & 7)) return false;
  if (g.epi == EPI_F32) {
    if (!g.ws) return false;
  } else if (g.epi == EPI_XENT_STATS) {
    if (!g.stats || !g.tz || !g.targets0) return false;
    if (g.C && ((g.ldc & 7) || (g.strideC & 7) || !aligned16(g.C))) return false;  // kept logits leave by TMA only
  } else {
    if (!g.C && g.epi != EPI_XENT_STATS) return false;
  }
  return true;
}

int device_sm_count() {
  static PerDevice pd;
  const int dev = PerDevice::current();
  if (dev >= 0 && pd.done[dev]) return pd.value[dev];
  int n = 0, cur = 0;
  cudaGetDevice(&cur);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, cur);
  if (n <= 0) n = 148;
  if (dev >= 0) { pd.value[dev] = n; pd.done[dev] = true; }
  return n;
}
static int num_sms() { return device_sm_count(); }

// Optional per-launch timing of the GEMM kernel (measurement aid, off by default).
namespace {
struct GemmProfile {
  bool on = false;
  std::vector<cudaEvent_t> ev;
  double flops = 0.0;
} g_prof;
}  // namespace

bool gemm_profiling() { return g_prof.on; }
extern "C" int32_t femto_profile_gemm(int32_t enable) {
  for (auto e : g_prof.ev) cudaEventDestroy(e);
  g_prof.ev.clear();
  g_prof.flops = 0.0;
  g_prof.on = enable != 0;
  return 0;
}
extern "C" int32_t femto_profile_gemm_report(double* h_ms, double* h_flops, int32_t* h_launches) {
  double ms = 0.0;
  for (size_t i = 0; i + 1 < g_prof.ev.size(); i += 2) {
    cudaEventSynchronize(g_prof.ev[i + 1]);
    float t = 0.f;
    cudaEventElapsedTime(&t, g_prof.ev[i], g_prof.ev[i + 1]);
    ms += t;
  }
  if (h_ms) *h_ms = ms;
  if (h_flops) *h_flops = g_prof.flops;
  if (h_launches) *h_launches = (int32_t)(g_prof.ev.size() / 2);
  return 0;
}

// ---- bounded-wait self test ---------------------------------------------------------------------------------------
// Runs the wait primitive of every warp-specialised kernel on a barrier that nothing will ever complete, with a
// small poll limit: the waiting thread must give up, raise the abort flag and status bit 2, the other role must see
// the flag and unwind, and the kernel must return normally (no trap, no hang).  result[0] = 1 when the waiter timed
// out, result[1] = 1 when the second role left through the abort flag.
namespace {
__global__ void k_bounded_wait_selftest(uint32_t limit, unsigned int* status, int* result) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); *abort_flag = 0; fence_barrier_init(); }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait_limit(&bar, 0, abort_flag, status, limit);
    result[0] = ok ? 0 : 1;
  } else if (threadIdx.x == 32) {
    // a second role waiting on the same dead barrier with the full limit: it must leave early through the abort flag
    const bool ok = mbar_wait(&bar, 0, abort_flag, nullptr);
    result[1] = (!ok && *abort_flag) ? 1 : 0;
  }
}
}  // namespace

extern "C" int32_t femto_selftest_bounded_wait(int32_t polls, int32_t* h_status, int32_t* h_result2) {
  if (polls <= 0 || !h_status || !h_result2) return femto_fail(FEMTO_ERR_ARG, "bad argument");
  unsigned int* status = nullptr;
  FEMTO_TRY(standalone_status(&status));
  int* result = nullptr;
  char* scratch = nullptr;
  FEMTO_TRY(standalone_scratch(256, &scratch));
  result = reinterpret_cast<int*>(scratch);
  CUDA_TRY(cudaMemset(result, 0, 2 * sizeof(int)));
  k_bounded_wait_selftest<<<1, 64>>>((uint32_t)polls, status, result);
  KERNEL_CHECK();
  CUDA_TRY(cudaDeviceSynchronize());                 // the kernel returned by itself
  unsigned int w = 0;
  CUDA_TRY(cudaMemcpy(&w, status, sizeof(w), cudaMemcpyDeviceToHost));
  CUDA_TRY(cudaMemset(status, 0, sizeof(w)));
  CUDA_TRY(cudaMemcpy(h_result2, result, 2 * sizeof(int), cudaMemcpyDeviceToHost));
  *h_status = (int32_t)w;
  return 0;
}

// 0 = one CTA per 128 x 256 tile, 1 = CTA pairs per 256 x 256 tile wherever the shape allows (the default).
static int g_pair_mode = -1;
extern "C" int32_t femto_gemm_pair_mode(int32_t mode) {
  const int old = g_pair_mode < 0 ? 1 : g_pair_mode;
  if (mode == 0 || mode == 1) g_pair_mode = mode;
  return old;
}

template <bool PAIR>
static int launch_tc(const GemmArgs& g, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const TcParams& p,
                     int grid, cudaStream_t s) {
  typedef Geo<PAIR> G;
  static PerDevice attr;
  const int dev = PerDevice::current();
  if (dev < 0 || !attr.done[dev]) {
    CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<true, true, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM_BYTES));
    CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<true, false, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM_BYTES));
    CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<false, true, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM_BYTES));
    CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<false, false, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM_BYTES));
    if (dev >= 0) attr.done[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(NTHREADS); cfg.stream = s;
  cfg.dynamicSmemBytes = G::SMEM_BYTES - (G::STAGES - p.stages) * G::STAGE_BYTES;
  static int pdl = -1;   // FEMTO_PDL=0 in the environment launches fully serialised (measurement aid)
  if (pdl < 0) { const char* e = getenv("FEMTO_PDL"); pdl = (e && e[0] == '0') ? 0 : 1; }
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = PAIR ? 2 : 1; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = pdl ? 2 : 1;
  cudaError_t e;
  if (g.a_kmajor && g.b_kmajor) e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<true, true, PAIR>, tmA, tmB, tmC, p);
  else if (g.a_kmajor) e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<true, false, PAIR>, tmA, tmB, tmC, p);
  else if (g.b_kmajor) e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<false, true, PAIR>, tmA, tmB, tmC, p);
  else e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<false, false, PAIR>, tmA, tmB, tmC, p);
  if (e != cudaSuccess) return femto_fail((int)e, "gemm_tc launch failed: %s", cudaGetErrorString(e));
  return 0;
}

int gemm_tc_bf16(const GemmArgs& g, cudaStream_t s) {
  if (!gemm_tc_supported(g)) return femto_fail(FEMTO_ERR_UNSUPPORTED, "gemm_tc: shape/alignment not supported");
  TcParams p;
  p.g = g;
  const int nb = g.batch;
  const int sms = num_sms();
  // CTA pairs need two row-tiles to share a B tile, and an M/N-contiguous operand to be expressible as 64-wide slabs
  CUtensorMap tmA, tmB;
  p.a_slabs = p.b_slabs = 0;
  if (g_pair_mode < 0) {   // first call: FEMTO_GEMM_PAIR=0 in the environment selects single-CTA tiles (measurement aid)
    const char* e = getenv("FEMTO_GEMM_PAIR");
    g_pair_mode = (e && e[0] == '0') ? 0 : 1;
  }
  bool pair = (g_pair_mode != 0) && g.M >= 2 * BM && sms >= 2;
  if (pair) {
    if (g.a_kmajor) pair = make_tmap_3d_bf16(&tmA, g.A, g.K, g.M, nb, g.lda, g.strideA, 64, BM) == 0;
    else pair = make_tmap_4d_slabs_bf16(&tmA, g.A, g.M, g.K, nb, g.lda, g.strideA, BK, BM / 64) == 0;
    if (pair) {
      if (g.b_kmajor) pair = make_tmap_3d_bf16(&tmB, g.B, g.K, g.N, nb, g.ldb, g.strideB, 64, BN / 2) == 0;
      else pair = make_tmap_4d_slabs_bf16(&tmB, g.B, g.N, g.K, nb, g.ldb, g.strideB, BK, BN / 128) == 0;
    }
    if (pair) { p.a_slabs = !g.a_kmajor; p.b_slabs = !g.b_kmajor; }
  }
  p.pair = pair ? 1 : 0;
  {
    // FEMTO_GEMM_STAGES in the environment shortens the operand ring (measurement aid)
    static int want = -1;
    if (want < 0) { const char* e = getenv("FEMTO_GEMM_STAGES"); want = e ? atoi(e) : 0; }
    const int full = pair ? Geo<true>::STAGES : Geo<false>::STAGES;
    p.stages = (want >= 2 && want <= full) ? want : (g.ring >= 2 && g.ring <= full) ? g.ring : full;
  }
  const int tile_m = pair ? 2 * BM : BM;
  const int workers = pair ? sms / 2 : sms;      // CTAs, or CTA pairs, that run at once
  p.tiles_m = cdiv(g.M, tile_m);
  p.tiles_n = cdiv(g.N, BN);
  p.kblocks = cdiv(g.K, BK);
  const int tiles = p.tiles_m * p.tiles_n * g.batch;
  int splits = 1;
  if (g.epi == EPI_F32 && tiles < 4 * workers) {
    // Pick the split count that minimises waves x k-blocks per unit PLUS what the partials cost: every split writes
    // and re-reads one fp32 copy of the result (8 bytes per element through HBM, the reduce pass not overlapped with
    // anything).  Both terms in units of one k-block of one worker, with round figures for the two rates.
    const size_t per_unit = (size_t)tile_m * BN * 4;
    const double kblock_s = 2.0 * tile_m * BN * BK / (1.3e15 / workers);
    static int charge = -1;
    if (charge < 0) { const char* e = getenv("FEMTO_SPLIT_COST"); charge = (e && e[0] == '0') ? 0 : 1; }
    const double per_split = charge ? 8.0 * g.M * (double)g.N * g.batch / 6.5e12 / kblock_s : 0.0;
    double best = (double)cdiv(tiles, workers) * p.kblocks;
    for (int sp = 2; sp <= 32 && sp <= p.kblocks; sp++) {
      if ((size_t)tiles * sp * per_unit > g.ws_bytes) break;
      const int kbp = cdiv(p.kblocks, sp);
      if ((sp - 1) * kbp >= p.kblocks) continue;
      const double cost = (double)cdiv((long long)tiles * sp, workers) * kbp + sp * per_split;
      if (cost < best) { best = cost; splits = sp; }
    }
  }
  p.splits = splits;
  p.kb_per_split = cdiv(p.kblocks, splits);
  p.total_units = tiles * splits;
  p.partial = reinterpret_cast<float*>(g.ws);

  if (!pair) {
    if (g.a_kmajor) FEMTO_TRY(make_tmap_3d_bf16(&tmA, g.A, g.K, g.M, nb, g.lda, g.strideA, 64, BM));
    else if (make_tmap_4d_slabs_bf16(&tmA, g.A, g.M, g.K, nb, g.lda, g.strideA, BK, BM / 64) == 0) p.a_slabs = 1;
    else FEMTO_TRY(make_tmap_3d_bf16(&tmA, g.A, g.M, g.K, nb, g.lda, g.strideA, 64, BK));
    if (g.b_kmajor) FEMTO_TRY(make_tmap_3d_bf16(&tmB, g.B, g.K, g.N, nb, g.ldb, g.strideB, 64, BN));
    else if (make_tmap_4d_slabs_bf16(&tmB, g.B, g.N, g.K, nb, g.ldb, g.strideB, BK, BN / 64) == 0) p.b_slabs = 1;
    else FEMTO_TRY(make_tmap_3d_bf16(&tmB, g.B, g.N, g.K, nb, g.ldb, g.strideB, 64, BK));
  }

  CUtensorMap tmC = tmA;
  p.tma_store = 0;
  const bool bf16_out = g.epi != EPI_F32 && (g.epi != EPI_XENT_STATS || g.C != nullptr);
  if (bf16_out && splits == 1 && (g.ldc & 7) == 0 && (g.strideC & 7) == 0 && aligned16(g.C)) {
    FEMTO_TRY(make_tmap_3d_bf16_sw(&tmC, g.C, g.N, g.M, nb, g.ldc, g.strideC, 64, 32, 3));
    p.tma_store = 1;
  }
  const int grid = pair ? 2 * std::min(p.total_units, workers) : std::min(p.total_units, sms);
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (g_prof.on) {
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaEventRecord(e0, s);
  }
  if (pair) FEMTO_TRY(launch_tc<true>(g, tmA, tmB, tmC, p, grid, s));
  else FEMTO_TRY(launch_tc<false>(g, tmA, tmB, tmC, p, grid, s));
  if (g_prof.on) {
    cudaEventRecord(e1, s);
    g_prof.ev.push_back(e0); g_prof.ev.push_back(e1);
    g_prof.flops += 2.0 * g.M * (double)g.N * g.K * g.batch;
  }
  KERNEL_CHECK();
  if (splits > 1) {
    gemm_tc_reduce_kernel<<<tiles * (pair ? 2 : 1) * 8, 256, 0, s>>>(p);
    KERNEL_CHECK();
  }
  return 0;
}
