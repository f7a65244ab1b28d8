// Prefill multi-LoRA kernels (bf16) on the Blackwell tensor cores: tcgen05.mma with TMEM
// accumulators, operands staged in shared memory by tiled TMA loads (no multicast), mbarrier
// pipelines between a TMA warp, an MMA-issuing thread and four epilogue warps.
//
// Tiling follows the token order, not the bucket arrays: block k owns rows [128k, 128k+128)
// of x / y. Inside a block, maximal runs of consecutive rows with the same slot (>= 0) are
// found from token_to_slot; in a prefill batch a block is one run, two at a request boundary.
// Each run is one M=128 MMA tile whose rows outside the run are computed and thrown away
// (masked in the epilogue), so rows with slot -1 are never written.
//
//   sgmv_shrink_kernel : tmp[s, rows, :] = sc * x[rows, :] . A_s[slot]^T        (K = in)
//   sgmv_expand_kernel : y[rows, cols]  += tmp[s, rows, :] . B_s[slot][cols]^T   (K = r)
// tmp [n, T, r_max] (bf16) lives in caller-provided scratch memory.
#pragma once

#include "tc_common.cuh"
#include "bgmv_fused.cuh"  // launch options shared by all kernels (programmatic dependent launch on / off)

namespace b200lora {

constexpr int kSgmvThreads = 192;   // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue
constexpr int kSgmvBM = 128;        // rows per block / MMA M
constexpr int kShrinkRows = 64;     // rows of x one shrink CTA owns (the upper half of its M = 128 tiles is idle)
constexpr int kSgmvBK = 64;         // K columns per shrink stage (one 128-byte swizzle row)
constexpr int kSgmvBN = 256;        // output columns per expand tile
constexpr int kSgmvShrinkMaxStages = 12; // the launch picks as many 64-column stages as fit into shared memory
constexpr int kSgmvExpandStages = 3;
constexpr int kSgmvAutoMinTokens = 512;  // IMPL_AUTO uses these kernels from this batch size on

struct SgmvArgs {
  __nv_bfloat16* y; int64_t y_ld;
  __nv_bfloat16* tmp;                       // [n, T, r_max]
  int T, in_dim, S, r_max, n;
  int out[B200_LORA_MAX_SLICES], col[B200_LORA_MAX_SLICES];
  const int32_t* token_to_slot;
  const float* scale_per_slot; float scaling;
  int zero_fill;                            // shrink: write zero rows for tokens without adapter
  int skip_clean;                           // expand: leave blocks in which every row has an adapter to tc_tile_kernel
  int shrink_gmax;                          // shrink: runs of a block whose K loops share one pass over x (set by the launch)
  int shrink_ring_bytes;                    // shrink: bytes of the TMA ring (set by the launch)
};

struct SgmvMaps {
  CUtensorMap x;                            // [T, in]            box 128 x 64
  CUtensorMap xs;                           // [T, in]            box  64 x 64 (shrink)
  CUtensorMap a[B200_LORA_MAX_SLICES];      // [S*r_max, in]      box r_max x 64
  CUtensorMap t;                            // [n*T, r_max]       box 128 x r_max
  CUtensorMap b[B200_LORA_MAX_SLICES];      // [S*out_s, r_max]   box 256 x r_max
};

// Runs of equal slot inside block `blk`, written to shared memory by thread 0.
// (table element types are the caller's: slot ids fit int16 for S <= 32767, row bounds 0..128 fit uint8)
template <typename TS, typename TR, int ROWS = kSgmvBM>
__device__ __forceinline__ void sgmv_find_runs(const int32_t* tts, int T, int S, int blk, TS* s_slot, TS* run_slot,
                                               TR* run_lo, TR* run_hi, int* nruns) {
  const int row0 = blk * ROWS;
  for (int i = threadIdx.x; i < ROWS; i += blockDim.x) {
    const int row = row0 + i;
    int sl = -1;
    if (row < T) sl = tts[row];
    (void)B200_IN_BOUNDS(sl >= -1 && sl < S);  // ids outside [-1, S) are treated as "no adapter"; the checked build reports them
    if (sl >= S || sl < -1) sl = -1;
    s_slot[i] = (TS)sl;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int n = 0, i = 0;
    while (i < ROWS) {
      const int sl = s_slot[i];
      if (sl < 0) { ++i; continue; }
      int j = i + 1;
      while (j < ROWS && s_slot[j] == sl) ++j;
      run_slot[n] = (TS)sl; run_lo[n] = (TR)i; run_hi[n] = (TR)j; ++n;
      i = j;
    }
    *nruns = n;
  }
  __syncthreads();
}

__device__ __forceinline__ void store_bf16x32(__nv_bfloat16* dst, const uint32_t (&v)[32], float sc, int ncols) {
  // v holds fp32 bit patterns of 32 consecutive columns; write the first `ncols` (multiple of 8)
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    if (q * 8 < ncols) {
      uint4 o;
      o.x = pack_bf16x2(__uint_as_float(v[8 * q + 0]) * sc, __uint_as_float(v[8 * q + 1]) * sc);
      o.y = pack_bf16x2(__uint_as_float(v[8 * q + 2]) * sc, __uint_as_float(v[8 * q + 3]) * sc);
      o.z = pack_bf16x2(__uint_as_float(v[8 * q + 4]) * sc, __uint_as_float(v[8 * q + 5]) * sc);
      o.w = pack_bf16x2(__uint_as_float(v[8 * q + 6]) * sc, __uint_as_float(v[8 * q + 7]) * sc);
      stg128(dst + 8 * q, o);
    }
  }
}

// Optional timeline of tuning builds: wall clock (ns) at entry / exit of every shrink CTA, SM clock at the
// k-steps of CTA 0's MMA thread.
#ifdef B200_TRACE
#define B200_SHRINK_TRACE_CTA(which)                                                        \
  if (threadIdx.x == 0 && blockIdx.x < 512) {                                               \
    unsigned long long t_;                                                                  \
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                  \
    g_b200_trace[4096 + 2 * blockIdx.x + (which)] = (long long)t_;                          \
  }
#define B200_SHRINK_TRACE_K(i) \
  if (blockIdx.x == 0 && (i) < 256) g_b200_trace[6144 + (i)] = clock64();
#else
#define B200_SHRINK_TRACE_CTA(which)
#define B200_SHRINK_TRACE_K(i)
#endif

// ============================================================================ shrink
__global__ void __launch_bounds__(kSgmvThreads, 1)
sgmv_shrink_kernel(const __grid_constant__ SgmvMaps maps, const SgmvArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ int s_slot[kSgmvBM], run_slot[kSgmvBM], run_lo[kSgmvBM], run_hi[kSgmvBM];
  __shared__ int nruns_s;
  __shared__ __align__(8) uint64_t bars[2 * kSgmvShrinkMaxStages + 2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int blk = blockIdx.x;
  const int r = a.r_max, n = a.n;
  B200_SHRINK_TRACE_CTA(0)
  // A CTA owns kShrinkRows = 64 rows of x: twice as many CTAs as 128-row blocks, so that most SMs of the GPU
  // stream x (a CTA's rate is bound by the bytes its ring keeps in flight). The MMAs stay M = 128: the x slot of a
  // stage has room for 128 rows, TMA fills the lower 64, the upper 64 hold stale bytes whose accumulator rows
  // (TMEM lanes 64..127) are never read.
  const uint32_t a_tile_bytes = (uint32_t)r * kSgmvBK * 2;
  const uint32_t x_tile_bytes = kSgmvBM * kSgmvBK * 2;
  const uint32_t x_load_bytes = kShrinkRows * kSgmvBK * 2;
  const uint32_t smem_base = (smem_u32(smem) + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (uint32_t)(kSgmvShrinkMaxStages + s); };
  const uint32_t acc_full = bar0 + 8u * (2 * kSgmvShrinkMaxStages);
  const uint32_t acc_empty = acc_full + 8u;
  int tmem_cols = 32;  // the last slice is read in 32-column chunks
  while (tmem_cols < (a.shrink_gmax * n - 1) * r + ((r + 31) & ~31)) tmem_cols *= 2;

  if (tid == 0) {
    for (int s = 0; s < kSgmvShrinkMaxStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, kShrinkRows);
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), (uint32_t)tmem_cols);
    tc_fence_before_sync();
  }
  sgmv_find_runs<int, int, kShrinkRows>(a.token_to_slot, a.T, a.S, blk, s_slot, run_slot, run_lo, run_hi, &nruns_s);  // has __syncthreads
  // Launched under programmatic dependent launch: everything above (barriers, TMEM, the run table from the index
  // metadata) may overlap the previous kernel of the stream; x is read and tmp written only from here on.
  griddep_wait();
  // Only now may the tile kernel that follows start: it reads x (and W) without waiting for anything, so it must
  // not run before the kernels ahead of this one are complete; it waits for this kernel before it reads tmp.
  griddep_launch_dependents();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  const int nruns = nruns_s;
  const int nk = a.in_dim / kSgmvBK;
  // The runs of a block (two at a request boundary) share ONE pass over x: every K step loads the x tile once
  // and one lora_A tile per run and slice, and the MMAs of run i accumulate into their own TMEM columns
  // [(i * n + s) * r, +r). Up to G runs per pass; the ring depth follows from the stage size of this block.
  const int G = min(a.shrink_gmax, max(nruns, 1));
  const uint32_t stage_bytes = x_tile_bytes + (uint32_t)(G * n) * a_tile_bytes;
  const int NS = min(kSgmvShrinkMaxStages, (int)((uint32_t)a.shrink_ring_bytes / stage_bytes));
  const int npass = (nruns + G - 1) / G;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&maps.xs);
      for (int s = 0; s < n; ++s) tma_prefetch_desc(&maps.a[s]);
      int st = 0, round = 0;
      for (int pi = 0; pi < npass; ++pi) {
        const int u0 = pi * G, g = min(G, nruns - u0);
        for (int kc = 0; kc < nk; ++kc) {
          if (round > 0) mbar_wait_bounded(empty_bar(st), (uint32_t)((round & 1) ^ 1), &abort_flag);
          const uint32_t base = smem_base + (uint32_t)st * stage_bytes;
          mbar_arrive_expect_tx(full_bar(st), x_load_bytes + (uint32_t)(g * n) * a_tile_bytes);
          tma_load_2d(base, &maps.xs, kc * kSgmvBK, blk * kShrinkRows, full_bar(st));
          for (int ui = 0; ui < g; ++ui) {
            const int slot = run_slot[u0 + ui];
            for (int s = 0; s < n; ++s)
              tma_load_2d(base + x_tile_bytes + (uint32_t)(ui * n + s) * a_tile_bytes, &maps.a[s], kc * kSgmvBK, slot * r,
                          full_bar(st));
          }
          if (++st == NS) { st = 0; ++round; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(kSgmvBM, r);
      int st = 0, round = 0;
      for (int pi = 0; pi < npass; ++pi) {
        const int g = min(G, nruns - pi * G);
        if (pi > 0) mbar_wait_bounded(acc_empty, (uint32_t)((pi - 1) & 1), &abort_flag);
        tc_fence_after_sync();
        for (int kc = 0; kc < nk; ++kc) {
          mbar_wait_bounded(full_bar(st), (uint32_t)(round & 1), &abort_flag);
          B200_SHRINK_TRACE_K(kc)
          tc_fence_after_sync();
          const uint32_t base = smem_base + (uint32_t)st * stage_bytes;
          const uint64_t xdesc = umma_smem_desc(base, 128);
          for (int q = 0; q < g * n; ++q) {  // q = run in pass * n + slice
            const uint64_t adesc = umma_smem_desc(base + x_tile_bytes + (uint32_t)q * a_tile_bytes, 128);
#pragma unroll
            for (int k4 = 0; k4 < kSgmvBK / 16; ++k4)
              umma_bf16(tmem_base + (uint32_t)(q * r), xdesc + 2u * k4, adesc + 2u * k4, idesc, (kc > 0 || k4 > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(st));  // stage reusable once these MMAs have read it
          if (++st == NS) { st = 0; ++round; }
        }
        umma_commit(acc_full);
      }
    }
  } else if ((warp & 3) < kShrinkRows / 32) {
    // epilogue: thread <-> row; a warp may only touch its own quarter of the 128 TMEM lanes (the warps of the
    // idle upper half have nothing to do)
    const int quarter = warp & 3;
    const int row_in_blk = quarter * 32 + lane;
    const int row = blk * kShrinkRows + row_in_blk;
    if (a.zero_fill && row < a.T && s_slot[row_in_blk] < 0) {
      for (int s = 0; s < n; ++s) {
        __nv_bfloat16* dst = a.tmp + ((int64_t)s * a.T + row) * r;
        for (int c = 0; c < r; c += 8) stg128(dst + c, make_uint4(0, 0, 0, 0));
      }
    }
    for (int pi = 0; pi < npass; ++pi) {
      const int u0 = pi * G, g = min(G, nruns - u0);
      mbar_wait_bounded(acc_full, (uint32_t)(pi & 1), &abort_flag);
      tc_fence_after_sync();
      for (int ui = 0; ui < g; ++ui) {
        const int u = u0 + ui;
        // (a TMEM load is a warp-wide operation on one column range: a warp whose 32 rows straddle two runs
        //  reads both runs' columns and every lane keeps the ones of its own run)
        const int lo_row = run_lo[u], hi_row = run_hi[u];
        if (hi_row <= quarter * 32 || lo_row >= quarter * 32 + 32) continue;  // warp-uniform: no row of this warp
        const bool mine = row_in_blk >= lo_row && row_in_blk < hi_row && row < a.T;
        const int slot = run_slot[u];
        const float sc = a.scaling * (a.scale_per_slot != nullptr ? a.scale_per_slot[slot] : 1.0f);
        for (int s = 0; s < n; ++s) {
          for (int c = 0; c < r; c += 32) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)((ui * n + s) * r + c), v);
            tmem_ld_wait();
            if (mine) store_bf16x32(a.tmp + ((int64_t)s * a.T + row) * r + c, v, sc, min(32, r - c));
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(acc_empty);
    }
  }
  __syncthreads();
  B200_SHRINK_TRACE_CTA(1)
  if (warp == 1) tmem_dealloc(tmem_base, (uint32_t)tmem_cols);
  if (tid == 0 && abort_flag != 0) atomicOr(&g_b200_status, kStatusWaitGaveUp);
}

// ============================================================================ expand
__global__ void __launch_bounds__(kSgmvThreads, 1)
sgmv_expand_kernel(const __grid_constant__ SgmvMaps maps, const SgmvArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ int s_slot[kSgmvBM], run_slot[kSgmvBM], run_lo[kSgmvBM], run_hi[kSgmvBM];
  __shared__ int nruns_s;
  __shared__ __align__(8) uint64_t bars[2 * kSgmvExpandStages + 4];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int blk = blockIdx.x, z = blockIdx.y, Z = gridDim.y;
  const int r = a.r_max, n = a.n;
  const uint32_t t_tile_bytes = (uint32_t)kSgmvBM * r * 2;
  const uint32_t b_tile_bytes = (uint32_t)kSgmvBN * r * 2;
  const uint32_t stage_bytes = t_tile_bytes + b_tile_bytes;
  const uint32_t smem_base = (smem_u32(smem) + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (uint32_t)(kSgmvExpandStages + s); };
  auto acc_full = [&](int b) { return bar0 + 8u * (uint32_t)(2 * kSgmvExpandStages + b); };
  auto acc_empty = [&](int b) { return bar0 + 8u * (uint32_t)(2 * kSgmvExpandStages + 2 + b); };
  constexpr int tmem_cols = 2 * kSgmvBN;  // two accumulator buffers

  if (tid == 0) {
    for (int s = 0; s < kSgmvExpandStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 128); }
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), (uint32_t)tmem_cols);
    tc_fence_before_sync();
  }
  sgmv_find_runs(a.token_to_slot, a.T, a.S, blk, s_slot, run_slot, run_lo, run_hi, &nruns_s);
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  int nruns = nruns_s;
  {
    // blocks in which every in-range row has an adapter are done by tc_tile_kernel when asked to
    const int nvalid = min(kSgmvBM, a.T - blk * kSgmvBM);
    int covered = 0;
    for (int u = 0; u < nruns; ++u) covered += run_hi[u] - run_lo[u];
    if (a.skip_clean && covered == nvalid) nruns = 0;
  }
  const int row_bytes = r * 2;  // 32 / 64 / 128: the swizzle span of both operand tiles

  // Jobs of this CTA, in the same order for all three roles:
  //   for run u, for slice s, for column tile j = z, z+Z, ... of the slice
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&maps.t);
      for (int s = 0; s < n; ++s) tma_prefetch_desc(&maps.b[s]);
      int st = 0, round = 0;
      for (int u = 0; u < nruns; ++u) {
        const int slot = run_slot[u];
        for (int s = 0; s < n; ++s) {
          const int ntile = (a.out[s] + kSgmvBN - 1) / kSgmvBN;
          for (int j = z; j < ntile; j += Z) {
            if (round > 0) mbar_wait_bounded(empty_bar(st), (uint32_t)((round & 1) ^ 1), &abort_flag);
            const uint32_t base = smem_base + (uint32_t)st * stage_bytes;
            mbar_arrive_expect_tx(full_bar(st), stage_bytes);
            tma_load_2d(base, &maps.t, 0, s * a.T + blk * kSgmvBM, full_bar(st));
            tma_load_2d(base + t_tile_bytes, &maps.b[s], 0, slot * a.out[s] + j * kSgmvBN, full_bar(st));
            if (++st == kSgmvExpandStages) { st = 0; ++round; }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(kSgmvBM, kSgmvBN);
      int st = 0, round = 0, job = 0;
      for (int u = 0; u < nruns; ++u) {
        for (int s = 0; s < n; ++s) {
          const int ntile = (a.out[s] + kSgmvBN - 1) / kSgmvBN;
          for (int j = z; j < ntile; j += Z, ++job) {
            const int buf = job & 1;
            if (job >= 2) mbar_wait_bounded(acc_empty(buf), (uint32_t)(((job >> 1) - 1) & 1), &abort_flag);
            mbar_wait_bounded(full_bar(st), (uint32_t)(round & 1), &abort_flag);
            tc_fence_after_sync();
            const uint32_t base = smem_base + (uint32_t)st * stage_bytes;
            const uint64_t tdesc = umma_smem_desc(base, row_bytes);
            const uint64_t bdesc = umma_smem_desc(base + t_tile_bytes, row_bytes);
            for (int k4 = 0; k4 < r / 16; ++k4)
              umma_bf16(tmem_base + (uint32_t)(buf * kSgmvBN), tdesc + 2u * k4, bdesc + 2u * k4, idesc, k4 > 0 ? 1u : 0u);
            umma_commit(empty_bar(st));
            umma_commit(acc_full(buf));
            if (++st == kSgmvExpandStages) { st = 0; ++round; }
          }
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int row_in_blk = quarter * 32 + lane;
    const int row = blk * kSgmvBM + row_in_blk;
    int job = 0;
    for (int u = 0; u < nruns; ++u) {
      const bool mine = row_in_blk >= run_lo[u] && row_in_blk < run_hi[u] && row < a.T;
      for (int s = 0; s < n; ++s) {
        const int ntile = (a.out[s] + kSgmvBN - 1) / kSgmvBN;
        for (int j = z; j < ntile; j += Z, ++job) {
          const int buf = job & 1;
          mbar_wait_bounded(acc_full(buf), (uint32_t)((job >> 1) & 1), &abort_flag);
          tc_fence_after_sync();
          const int c0 = j * kSgmvBN;
          __nv_bfloat16* yrow = a.y + (int64_t)row * a.y_ld + a.col[s] + c0;
          for (int c = 0; c < kSgmvBN; c += 32) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kSgmvBN + c), v);
            tmem_ld_wait();
            if (mine) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                if (c0 + c + 8 * q < a.out[s]) {
                  uint4 yv = ldg128(yrow + c + 8 * q);
                  yv.x = add_bf16x2(yv.x, __uint_as_float(v[8 * q + 0]), __uint_as_float(v[8 * q + 1]));
                  yv.y = add_bf16x2(yv.y, __uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]));
                  yv.z = add_bf16x2(yv.z, __uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]));
                  yv.w = add_bf16x2(yv.w, __uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]));
                  stg128(yrow + c + 8 * q, yv);
                }
              }
            }
          }
          tc_fence_before_sync();
          mbar_arrive(acc_empty(buf));
        }
      }
    }
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, (uint32_t)tmem_cols);
  if (tid == 0 && abort_flag != 0) atomicOr(&g_b200_status, kStatusWaitGaveUp);
}

// ============================================================================ host side
struct SgmvProblem {
  void* y; int64_t y_ld; const void* x; int64_t x_ld;
  int T, in_dim, S, r_max;
  SliceTable st;
  const float* scale_per_slot; const int32_t* token_to_slot; float scaling;
};

inline size_t sgmv_workspace_bytes(int T, int n_slices, int r_max) {
  // tmp [n, T, r_max] bf16, plus one 128-row tile of slack so the last TMA box stays inside the allocation
  return ((size_t)n_slices * (size_t)T + kSgmvBM) * (size_t)r_max * 2 + 1024;
}

// `with_x` / `with_b`: which of the two halves the caller runs (shrink reads x and lora_A, expand reads tmp and lora_B)
inline bool sgmv_supported(const SgmvProblem& b, const char** why, bool with_x = true, bool with_b = true) {
  const char* dummy;
  if (why == nullptr) why = &dummy;
  int n = 0;
  for (int s = 0; s < b.st.n; ++s) n += b.st.out[s] > 0;
  if (n == 0) { *why = "no active slice"; return false; }
  if (b.r_max != 16 && b.r_max != 32 && b.r_max != 64) { *why = "r_max must be 16, 32 or 64"; return false; }
  if (n * b.r_max > 512) { *why = "n_slices * r_max exceeds the 512 TMEM columns"; return false; }
  if (with_x) {
    if (b.in_dim % kSgmvBK != 0) { *why = "in_dim must be a multiple of 64"; return false; }
    if (b.x_ld % 8 != 0 || (reinterpret_cast<uintptr_t>(b.x) & 15u)) { *why = "x must be 16-byte aligned with a row stride that is a multiple of 8"; return false; }
  }
  if (with_b && (b.y_ld % 8 != 0 || (reinterpret_cast<uintptr_t>(b.y) & 15u))) { *why = "y must be 16-byte aligned with a row stride that is a multiple of 8"; return false; }
  for (int s = 0; s < b.st.n; ++s) {
    if (b.st.out[s] == 0) continue;
    if (with_b && (b.st.out[s] % 8 != 0 || b.st.col[s] % 8 != 0)) { *why = "slice widths / offsets must be multiples of 8"; return false; }
    if ((with_x && (reinterpret_cast<uintptr_t>(b.st.a[s]) & 15u)) || (with_b && (reinterpret_cast<uintptr_t>(b.st.b[s]) & 15u))) {
      *why = "slabs must be 16-byte aligned";
      return false;
    }
  }
  return true;
}

// Launch arguments and tensor maps over an intermediate `tmp` [n, T, r_max] (bf16, 16-byte aligned) that holds
// `tmp_rows` rows: rows beyond that are neither written nor read (the maps clip).
inline int sgmv_prepare_tmp(const SgmvProblem& b, void* tmp, uint64_t tmp_rows, bool with_x, bool with_b, SgmvMaps* maps,
                            SgmvArgs* args) {
  const char* why = nullptr;
  if (!sgmv_supported(b, &why, with_x, with_b)) return fail(B200_LORA_EUNSUPPORTED, "prefill kernels: %s", why);
  if (tmp == nullptr || (reinterpret_cast<uintptr_t>(tmp) & 15u)) return fail(B200_LORA_EINVAL, "prefill kernels: the intermediate must be 16-byte aligned");
  SgmvArgs a = {};
  a.n = 0;
  const void* slab_a[B200_LORA_MAX_SLICES];
  const void* slab_b[B200_LORA_MAX_SLICES];
  for (int s = 0; s < b.st.n; ++s) {
    if (b.st.out[s] == 0) continue;
    slab_a[a.n] = b.st.a[s]; slab_b[a.n] = b.st.b[s];
    a.out[a.n] = b.st.out[s]; a.col[a.n] = b.st.col[s];
    ++a.n;
  }
  a.y = static_cast<__nv_bfloat16*>(b.y); a.y_ld = b.y_ld;
  a.tmp = static_cast<__nv_bfloat16*>(tmp);
  a.T = b.T; a.in_dim = b.in_dim; a.S = b.S; a.r_max = b.r_max;
  a.token_to_slot = b.token_to_slot; a.scale_per_slot = b.scale_per_slot; a.scaling = b.scaling;
  a.zero_fill = 0;
  if (int rc = make_tmap_2d(&maps->t, a.tmp, tmp_rows, (uint64_t)b.r_max, (uint64_t)b.r_max, kSgmvBM, (uint32_t)b.r_max)) return rc;
  if (with_x) {
    if (int rc = make_tmap_2d(&maps->x, b.x, (uint64_t)b.T, (uint64_t)b.in_dim, (uint64_t)b.x_ld, kSgmvBM, kSgmvBK)) return rc;
    if (int rc = make_tmap_2d(&maps->xs, b.x, (uint64_t)b.T, (uint64_t)b.in_dim, (uint64_t)b.x_ld, kShrinkRows, kSgmvBK)) return rc;
  } else {
    maps->x = maps->xs = maps->t;  // never dereferenced by the expand half
  }
  for (int s = 0; s < a.n; ++s) {
    if (with_x) {
      if (int rc = make_tmap_2d(&maps->a[s], slab_a[s], (uint64_t)b.S * b.r_max, (uint64_t)b.in_dim, (uint64_t)b.in_dim, (uint32_t)b.r_max, kSgmvBK)) return rc;
    } else {
      maps->a[s] = maps->t;
    }
    if (with_b) {
      if (int rc = make_tmap_2d(&maps->b[s], slab_b[s], (uint64_t)b.S * a.out[s], (uint64_t)b.r_max, (uint64_t)b.r_max, kSgmvBN, (uint32_t)b.r_max)) return rc;
    } else {
      maps->b[s] = maps->t;
    }
  }
  for (int s = a.n; s < B200_LORA_MAX_SLICES; ++s) { maps->a[s] = maps->a[0]; maps->b[s] = maps->b[0]; }
  *args = a;
  return B200_LORA_OK;
}

// Builds the launch arguments and tensor maps shared by the two kernels, the intermediate in caller-provided scratch.
inline int sgmv_prepare(const SgmvProblem& b, void* workspace, size_t workspace_bytes, SgmvMaps* maps, SgmvArgs* args) {
  int n = 0;
  for (int s = 0; s < b.st.n; ++s) n += b.st.out[s] > 0;
  const size_t need = sgmv_workspace_bytes(b.T, std::max(n, 1), b.r_max);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(B200_LORA_EWORKSPACE, "prefill kernels need %zu bytes of scratch, got %zu", need, workspace_bytes);
  uintptr_t ws = (reinterpret_cast<uintptr_t>(workspace) + 1023) & ~(uintptr_t)1023;
  return sgmv_prepare_tmp(b, reinterpret_cast<void*>(ws), (uint64_t)n * b.T + kSgmvBM, true, true, maps, args);
}

inline int sgmv_set_smem(const void* kernel, size_t bytes) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return fail(B200_LORA_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  return B200_LORA_OK;
}

inline int sgmv_launch_shrink(const SgmvMaps& maps, const SgmvArgs& a_in, cudaStream_t stream) {
  SgmvArgs a = a_in;
  // One CTA per SM streams its 128 rows of x through a ring that fills the shared memory of the SM: the more
  // bytes in flight, the better. Up to 4 runs of a block share a pass, as long as their accumulators fit into
  // the 512 TMEM columns and three stages of that size fit into the ring.
  const size_t ring = 216 * 1024;
  const size_t x_tile = kSgmvBM * kSgmvBK * 2, a_tiles = (size_t)a.n * a.r_max * kSgmvBK * 2;
  int gmax = 1;
  for (int g = 2; g <= 4; ++g) {
    const int cols = (g * a.n - 1) * a.r_max + ((a.r_max + 31) & ~31);
    if (cols <= 512 && ring / (x_tile + g * a_tiles) >= 3) gmax = g;
  }
  a.shrink_gmax = gmax;
  a.shrink_ring_bytes = (int)ring;
  const size_t smem = ring + 1024;
  if (int rc = sgmv_set_smem(reinterpret_cast<const void*>(sgmv_shrink_kernel), smem)) return rc;
  const int nblk = (a.T + kShrinkRows - 1) / kShrinkRows;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)nblk, 1, 1);
  cfg.blockDim = dim3(kSgmvThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = bgmv_options().pdl ? 1 : 0;  // B200_LORA_OPT_PDL = 0: strict stream order (the waits in the kernel are then no-ops)
  cudaError_t e = cudaLaunchKernelEx(&cfg, sgmv_shrink_kernel, maps, a);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(B200_LORA_ECUDA, "sgmv_shrink_kernel launch: %s", cudaGetErrorString(e));
  }
  return B200_LORA_OK;
}

inline int sgmv_launch_expand(const SgmvMaps& maps, const SgmvArgs& a, cudaStream_t stream) {
  const size_t smem = (size_t)kSgmvExpandStages * ((size_t)kSgmvBM * a.r_max * 2 + (size_t)kSgmvBN * a.r_max * 2) + 1024;
  if (int rc = sgmv_set_smem(reinterpret_cast<const void*>(sgmv_expand_kernel), smem)) return rc;
  const int nblk = (a.T + kSgmvBM - 1) / kSgmvBM;
  int max_tiles = 1;
  for (int s = 0; s < a.n; ++s) max_tiles = std::max(max_tiles, (a.out[s] + kSgmvBN - 1) / kSgmvBN);
  int Z = std::max(1, std::min(max_tiles, (2 * 148 + nblk - 1) / nblk));
  sgmv_expand_kernel<<<dim3(nblk, Z), kSgmvThreads, smem, stream>>>(maps, a);
  return check_launch("sgmv_expand_kernel");
}

inline int sgmv_launch(const SgmvProblem& b, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  SgmvMaps maps;
  SgmvArgs args;
  if (int rc = sgmv_prepare(b, workspace, workspace_bytes, &maps, &args)) return rc;
  if (int rc = sgmv_launch_shrink(maps, args, stream)) return rc;
  return sgmv_launch_expand(maps, args, stream);
}

}  // namespace b200lora
