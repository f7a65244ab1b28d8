// Tensor-core tile kernel shared by the fused "base GEMM + LoRA" linear and by the fast
// path of the prefill expand (bf16, tcgen05.mma, TMEM accumulators, tiled TMA in and out).
//
// Output tile = 128 rows x 256 columns of the packed output y. For each tile the CTA runs
//   LINEAR : K loop over `in` with (x tile, W tile) stages               -> D  = x . W^T
//            then one extra stage per (run of equal slot, LoRA slice that intersects the tile):
//            (tmp_s tile with the rows outside the run zeroed, B_s[slot] rows) -> D += tmp_s . B_s^T
//            epilogue: (+ bias) -> bf16 -> shared memory -> TMA store.           y  = D
//   EXPAND : only the LoRA stages                                          -> D  = sum of deltas
//            epilogue: bf16 -> shared memory -> TMA reduce-add.                  y += D
// so the LoRA delta costs r/16 more MMAs on an accumulator that is already in TMEM, and the
// activation is neither written back nor re-read for it. The reduce-add is performed once per
// element at the L2 (deterministic).
//
// Rows of a block may use different slots (request boundaries): the mask warp zeroes, in the
// shared-memory copy of tmp, the rows that do not belong to the run whose B is being
// multiplied, so every row only receives its own adapter's delta. Rows without adapter get a
// zero delta: exact in LINEAR mode (y is stored, the base result is unchanged). In EXPAND mode
// their staged delta is NEGATIVE zero: x + (-0.0) == x bit for bit for every x, both zeros and
// denormals included (the reduce-add does not flush), whereas +0.0 would turn a -0.0 into +0.0.
#pragma once

#include "sgmv_tc.cuh"

namespace b200lora {

constexpr int kTileThreads = 224;  // warp 0 TMA, warp 1 MMA + TMEM owner, warps 2-5 epilogue, warp 6 row mask
constexpr int kTileSMs = 148;      // SMs of a B200: one persistent CTA each
constexpr int kTileMaxSeg = 3;     // row blocks one CTA's tile range may touch
#ifndef TC_TILE_Y_PREFETCH
#define TC_TILE_Y_PREFETCH 1  // reduce-add mode: tiles by which the L2 prefetch of y runs ahead (0 = off)
#endif
#ifndef B200_GEMM_STAGES
#define B200_GEMM_STAGES 4
#endif
#ifndef B200_GEMM_OUTBUFS
#define B200_GEMM_OUTBUFS 2
#endif
constexpr int kGemmStages = B200_GEMM_STAGES;
constexpr int kGemmStageBytes = kSgmvBM * kSgmvBK * 2 + kSgmvBN * kSgmvBK * 2;  // 48 KB: x tile + W tile
constexpr int kGemmOutChunk = 64;                                               // columns per TMA store box
constexpr int kGemmOutBufs = B200_GEMM_OUTBUFS;
constexpr int kGemmOutBufBytes = kSgmvBM * kGemmOutChunk * 2;                   // 16 KB

struct GemmArgs {
  int T, in_dim, n_total;          // rows, base K (0 in EXPAND mode), packed output width
  const __nv_bfloat16* bias;       // [n_total] or null (LINEAR)
  int S, r_max, n;
  int out[B200_LORA_MAX_SLICES], col[B200_LORA_MAX_SLICES];
  const int32_t* token_to_slot;
  int expand_mode;                 // 0 = LINEAR (store), 1 = EXPAND (reduce-add, blocks without -1 rows)
  int lora;                        // LINEAR: add the LoRA stages
  int overwrite;                   // EXPAND: store the delta tiles (-0.0 in rows without adapter) instead of adding them
  // Programmatic dependent launch: the kernel may start while the previous kernel of the stream still runs.
  // 1 = that kernel is this library's shrink (launched the ordinary way, so everything before it is complete, and
  //     it writes nothing but tmp): only the first load of tmp waits for it; the set-up, and in LINEAR mode the base
  //     GEMM of the first tiles, overlap it.
  // 0 = unknown predecessor: the first load of anything waits.
  int after_shrink;
  __nv_bfloat16* y; int64_t y_ld;  // plain view of the output beside its tensor map (L2 prefetch of the rows a reduce-add will touch)
};

struct GemmMaps {
  CUtensorMap x;                            // [T, in]           box 128 x 64
  CUtensorMap w;                            // [n_total, in]     box 256 x 64
  CUtensorMap t;                            // [n*T(+128), r]    box 128 x r
  CUtensorMap b[B200_LORA_MAX_SLICES];      // [S*out_s, r]      box 256 x r
  CUtensorMap y;                            // [T, n_total]      box 128 x 64 (store / reduce)
};

// L2 cache policies: the output is written once and not read again by this kernel (evict first),
// the weight tiles are re-read by every row block (evict last).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst_smem, const CUtensorMap* tmap, int c0, int c1, uint32_t bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(dst_smem), "l"(tmap), "r"(c0), "r"(c1), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d_hint(const CUtensorMap* tmap, uint32_t src_smem, int c0, int c1, uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;" ::"l"(tmap),
               "r"(src_smem), "r"(c0), "r"(c1), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, uint32_t src_smem, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap),
               "r"(src_smem), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* tmap, uint32_t src_smem, int c0, int c1) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap),
               "r"(src_smem), "r"(c0), "r"(c1)
               : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Optional timeline (SM clock) of CTA 0, compiled in only for tuning builds.
#ifdef B200_TRACE
#define B200_TILE_TRACE(idx) \
  if (blockIdx.x == 0 && (idx) < 1024 * 32) g_b200_trace[(idx)] = clock64();
// wall clock (ns) at entry / exit of every CTA
#define B200_TILE_TRACE_CTA(which)                                                          \
  if (threadIdx.x == 0) {                                                                   \
    unsigned long long t_;                                                                  \
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                  \
    g_b200_trace[2048 + 2 * blockIdx.x + (which)] = (long long)t_;                          \
  }
#else
#define B200_TILE_TRACE(idx)
#define B200_TILE_TRACE_CTA(which)
#endif

__global__ void __launch_bounds__(kTileThreads, 1)
tc_tile_kernel(const __grid_constant__ GemmMaps maps, const GemmArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  // run tables of the (at most kTileMaxSeg) row blocks this CTA's tile range touches; compact types:
  // the stages leave no room for more than 3 KB of static shared memory
  __shared__ int16_t s_slot[kTileMaxSeg][kSgmvBM], run_slot[kTileMaxSeg][kSgmvBM];
  __shared__ uint8_t run_lo[kTileMaxSeg][kSgmvBM], run_hi[kTileMaxSeg][kSgmvBM];
  __shared__ int seg_nruns[kTileMaxSeg];
  __shared__ __align__(8) uint64_t bars[3 * kGemmStages + 4];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = a.r_max, n = a.n;
  B200_TILE_TRACE_CTA(0)
  // the next kernel of the stream, if it was launched as a programmatic dependent (this library's shrink and decode
  // kernels are), may set itself up now; those kernels wait for this one before they touch activations or scratch
  griddep_launch_dependents();
  // Persistent schedule: the output tiles, numbered row block major (id = blk * ntile_all + j), are
  // dealt to the CTAs in equal contiguous ranges, so every SM gets the same number of tiles and a CTA
  // changes row block at most kTileMaxSeg - 1 times.
  const int ntile_all = (a.n_total + kSgmvBN - 1) / kSgmvBN;
  const int nblk_all = (a.T + kSgmvBM - 1) / kSgmvBM;
  const int total_tiles = nblk_all * ntile_all;
  const int per_cta = (total_tiles + (int)gridDim.x - 1) / (int)gridDim.x;
  const int t_begin = min((int)blockIdx.x * per_cta, total_tiles), t_end = min(t_begin + per_cta, total_tiles);
  const int blk_first = t_begin / ntile_all;
  const int nseg = t_end > t_begin ? (t_end - 1) / ntile_all - blk_first + 1 : 0;  // <= kTileMaxSeg (host)
  // The stages and output buffers fill the whole dynamic allocation (no alignment slack fits beside
  // four 48 KB stages), so the 1024-byte alignment the swizzled tiles need must come from the
  // declaration above; a base that is not aligned is reported instead of used.
  const uint32_t smem_base = smem_u32(smem);
  if ((smem_base & 1023u) != 0) {
    if (tid == 0) atomicOr(&g_b200_status, kStatusBadSmemBase);
    return;
  }
  const uint32_t out_base = smem_base + kGemmStages * kGemmStageBytes;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (uint32_t)(kGemmStages + s); };
  auto masked_bar = [&](int s) { return bar0 + 8u * (uint32_t)(2 * kGemmStages + s); };
  auto acc_full = [&](int b) { return bar0 + 8u * (uint32_t)(3 * kGemmStages + b); };
  auto acc_empty = [&](int b) { return bar0 + 8u * (uint32_t)(3 * kGemmStages + 2 + b); };
  constexpr int tmem_cols = 2 * kSgmvBN;

  if (tid == 0) {
    // a stage is free again once the MMA thread (tcgen05.commit) AND the mask warp are past it
    for (int s = 0; s < kGemmStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 2); mbar_init(masked_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 128); }
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), (uint32_t)tmem_cols);
    tc_fence_before_sync();
  }
  const bool with_runs = a.token_to_slot != nullptr && (a.lora || a.expand_mode);
  for (int sg = 0; sg < nseg; ++sg) {
    if (with_runs) {
      sgmv_find_runs(a.token_to_slot, a.T, a.S, blk_first + sg, s_slot[sg], run_slot[sg], run_lo[sg], run_hi[sg], &seg_nruns[sg]);
    } else if (tid == 0) {
      seg_nruns[sg] = 0;
    }
  }
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  const int nk = a.expand_mode ? 0 : a.in_dim / kSgmvBK;
  // tiles [ja, jb) of segment sg; EXPAND mode has nothing to add to a block without any adapter row
  auto seg_range = [&](int sg, int& blk, int& ja, int& jb, int& nruns) {
    blk = blk_first + sg;
    nruns = seg_nruns[sg];
    ja = max(t_begin - blk * ntile_all, 0);
    jb = min(t_end - blk * ntile_all, ntile_all);
    if (a.expand_mode && nruns == 0 && !a.overwrite) jb = ja;
  };
  const int row_bytes = r * 2;
  const uint32_t t_tile_bytes = (uint32_t)kSgmvBM * r * 2, b_tile_bytes = (uint32_t)kSgmvBN * r * 2;

  // The four roles walk the same stage sequence:
  //   for tile j: [nk base stages], then for run u, for slice s intersecting the tile: one LoRA stage
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&maps.x); tma_prefetch_desc(&maps.w); tma_prefetch_desc(&maps.t); tma_prefetch_desc(&maps.y);
      const uint64_t w_policy = l2_policy_evict_last();
      int st = 0, round = 0;
      bool waited = false;
      if (!a.after_shrink) { griddep_wait(); waited = true; }
      for (int sg = 0; sg < nseg; ++sg) {
      int blk, ja, jb, nruns;
      seg_range(sg, blk, ja, jb, nruns);
      for (int j = ja; j < jb; ++j) {
        for (int kc = 0; kc < nk; ++kc) {
          if (round > 0) mbar_wait_bounded(empty_bar(st), (uint32_t)((round & 1) ^ 1), &abort_flag);
          const uint32_t base = smem_base + (uint32_t)st * kGemmStageBytes;
          mbar_arrive_expect_tx(full_bar(st), kGemmStageBytes);
          tma_load_2d(base, &maps.x, kc * kSgmvBK, blk * kSgmvBM, full_bar(st));
          tma_load_2d_hint(base + kSgmvBM * kSgmvBK * 2, &maps.w, kc * kSgmvBK, j * kSgmvBN, full_bar(st), w_policy);
          if (++st == kGemmStages) { st = 0; ++round; }
        }
        for (int u = 0; u < nruns; ++u) {
          const int slot = run_slot[sg][u];
          for (int s = 0; s < n; ++s) {
            const int lo = max(a.col[s], j * kSgmvBN), hi = min(a.col[s] + a.out[s], (j + 1) * kSgmvBN);
            if (lo >= hi) continue;
            if (round > 0) mbar_wait_bounded(empty_bar(st), (uint32_t)((round & 1) ^ 1), &abort_flag);
            if (!waited) { griddep_wait(); waited = true; }  // tmp is final from here on
            const uint32_t base = smem_base + (uint32_t)st * kGemmStageBytes;
            mbar_arrive_expect_tx(full_bar(st), t_tile_bytes + b_tile_bytes);
            tma_load_2d(base, &maps.t, 0, s * a.T + blk * kSgmvBM, full_bar(st));
            tma_load_2d(base + t_tile_bytes, &maps.b[s], 0, slot * a.out[s] + (lo - a.col[s]), full_bar(st));
            B200_TILE_TRACE(768 + min(j - ja, 63) + 64 * sg)
            if (++st == kGemmStages) { st = 0; ++round; }
          }
        }
      }
      }
    }
  } else if (warp == 6) {
    // mask warp: zero the tmp rows outside the current run, then hand the stage to the MMA thread
    int st = 0, round = 0;
    for (int sg = 0; sg < nseg; ++sg) {
    int blk, ja, jb, nruns;
    seg_range(sg, blk, ja, jb, nruns);
    for (int j = ja; j < jb; ++j) {
      // (the masked barrier of a stage completes one phase per LoRA use of that stage; the MMA
      //  thread keeps the same per-stage phase bits)
      // Base stages need no masking, but their full barriers are still waited for: a waiter that
      // skipped phases could no longer tell phase k from phase k-2 by parity.
      for (int kc = 0; kc < nk; ++kc) {
        mbar_wait_bounded(full_bar(st), (uint32_t)(round & 1), &abort_flag);
        if (lane == 0) mbar_arrive(empty_bar(st));
        if (++st == kGemmStages) { st = 0; ++round; }
      }
      for (int u = 0; u < nruns; ++u) {
        const int lo_row = run_lo[sg][u], hi_row = run_hi[sg][u];
        for (int s = 0; s < n; ++s) {
          const int lo = max(a.col[s], j * kSgmvBN), hi = min(a.col[s] + a.out[s], (j + 1) * kSgmvBN);
          if (lo >= hi) continue;
          mbar_wait_bounded(full_bar(st), (uint32_t)(round & 1), &abort_flag);
          if (lo_row > 0 || hi_row < kSgmvBM) {
            // only the rows outside the run are visited: `chunks` lanes per row (its 16-byte pieces; the swizzle
            // only permutes them inside the row), 32 / chunks rows per step
            const uint32_t base = smem_base + (uint32_t)st * kGemmStageBytes;
            const int chunks = row_bytes >> 4;
            const int rows_per_step = 32 / chunks, sub = lane / chunks;
            const uint32_t piece = (uint32_t)(lane - sub * chunks) * 16u;
            for (int row = sub; row < lo_row; row += rows_per_step)
              asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(base + (uint32_t)(row * row_bytes) + piece), "r"(0u) : "memory");
            for (int row = hi_row + sub; row < kSgmvBM; row += rows_per_step)
              asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(base + (uint32_t)(row * row_bytes) + piece), "r"(0u) : "memory");
            fence_proxy_async_smem();
          }
          __syncwarp();
          if (lane == 0) { mbar_arrive(masked_bar(st)); mbar_arrive(empty_bar(st)); }
          if (++st == kGemmStages) { st = 0; ++round; }
        }
      }
    }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_base = umma_idesc_bf16(kSgmvBM, kSgmvBN);
      int st = 0, round = 0, job = 0;
      uint32_t mphase = 0;  // bit st: parity of the next phase of masked_bar(st)
      for (int sg = 0; sg < nseg; ++sg) {
      int blk, ja, jb, nruns;
      seg_range(sg, blk, ja, jb, nruns);
      for (int j = ja; j < jb; ++j, ++job) {
        const int buf = job & 1;
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kSgmvBN);
        if (job >= 2) mbar_wait_bounded(acc_empty(buf), (uint32_t)(((job >> 1) - 1) & 1), &abort_flag);
        B200_TILE_TRACE(512 + 4 * min(job, 31) + 0)
        tc_fence_after_sync();
        for (int kc = 0; kc < nk; ++kc) {
          mbar_wait_bounded(full_bar(st), (uint32_t)(round & 1), &abort_flag);
          tc_fence_after_sync();
          const uint32_t base = smem_base + (uint32_t)st * kGemmStageBytes;
          const uint64_t xdesc = umma_smem_desc(base, 128);
          const uint64_t wdesc = umma_smem_desc(base + kSgmvBM * kSgmvBK * 2, 128);
#pragma unroll
          for (int k4 = 0; k4 < kSgmvBK / 16; ++k4)
            umma_bf16(d_tmem, xdesc + 2u * k4, wdesc + 2u * k4, idesc_base, (kc > 0 || k4 > 0) ? 1u : 0u);
          umma_commit(empty_bar(st));
          if (++st == kGemmStages) { st = 0; ++round; }
        }
        uint32_t started = 0;  // bit s: the D columns of slice s already hold a partial sum
        for (int u = 0; u < nruns; ++u) {
          for (int s = 0; s < n; ++s) {
            const int lo = max(a.col[s], j * kSgmvBN), hi = min(a.col[s] + a.out[s], (j + 1) * kSgmvBN);
            if (lo >= hi) continue;
            mbar_wait_bounded(masked_bar(st), (mphase >> st) & 1u, &abort_flag);
            B200_TILE_TRACE(512 + 4 * min(job, 31) + 1)
            mphase ^= 1u << st;
            tc_fence_after_sync();
            const uint32_t base = smem_base + (uint32_t)st * kGemmStageBytes;
            const uint64_t tdesc = umma_smem_desc(base, row_bytes);
            const uint64_t bdesc = umma_smem_desc(base + t_tile_bytes, row_bytes);
            const uint32_t idesc = umma_idesc_bf16(kSgmvBM, (hi - lo + 15) & ~15);
            const bool fresh = nk == 0 && ((started >> s) & 1u) == 0;
            for (int k4 = 0; k4 < r / 16; ++k4)
              umma_bf16(d_tmem + (uint32_t)(lo - j * kSgmvBN), tdesc + 2u * k4, bdesc + 2u * k4, idesc,
                        (fresh && k4 == 0) ? 0u : 1u);
            started |= 1u << s;
            umma_commit(empty_bar(st));
            if (++st == kGemmStages) { st = 0; ++round; }
          }
        }
        umma_commit(acc_full(buf));
        B200_TILE_TRACE(512 + 4 * min(job, 31) + 2)
      }
      }
    }
  } else if (warp >= 2 && warp <= 5) {
    // epilogue warps: thread <-> row of the tile
    const int quarter = warp & 3;
    const int row_in_blk = quarter * 32 + lane;
    const int etid = tid - 64;  // 0..127
    int job = 0, chunk_no = 0;
    for (int sg = 0; sg < nseg; ++sg) {
    int blk, ja, jb, nruns;
    seg_range(sg, blk, ja, jb, nruns);
    // EXPAND mode: this thread's row has no adapter -> its delta is -0.0 (see the header comment)
    const bool neg_zero_row = a.expand_mode && s_slot[sg][row_in_blk] < 0;
    for (int j = ja; j < jb; ++j, ++job) {
      const int buf = job & 1;
#if TC_TILE_Y_PREFETCH > 0
      // The reduce-add reads y at the L2 in 128-byte row pieces (64-column boxes). Each thread asks for its row of the
      // tile that comes TC_TILE_Y_PREFETCH tiles later, all 256 columns in one piece: the DRAM reads become 512-byte
      // bursts that are over before the reductions arrive (one tile ahead measured best: 108 instead of 119 us on a
      // 8172 x 12288 output; two tiles 112, three 119, four 125).
      if (a.expand_mode && !a.overwrite) {
        const int cur = blk * ntile_all + j;
        for (int t = (job == 0 ? cur : cur + TC_TILE_Y_PREFETCH); t <= cur + TC_TILE_Y_PREFETCH && t < t_end; ++t) {
          const int pb = t / ntile_all, pj = t - pb * ntile_all;
          const int prow = pb * kSgmvBM + row_in_blk, pcol = pj * kSgmvBN;
          const int pcols = min(kSgmvBN, a.n_total - pcol);
          if (prow < a.T && pcols > 0) bulk_prefetch_l2(a.y + (int64_t)prow * a.y_ld + pcol, (uint32_t)pcols * 2u);
        }
      }
#endif
      mbar_wait_bounded(acc_full(buf), (uint32_t)((job >> 1) & 1), &abort_flag);
      if (etid == 0) { B200_TILE_TRACE(16 * min(job, 31) + 0) }
      tc_fence_after_sync();
      for (int c = 0; c < kSgmvBN; c += kGemmOutChunk, ++chunk_no) {
        const int col0 = j * kSgmvBN + c;
        if (col0 >= a.n_total) break;  // uniform over the CTA
        const uint32_t obuf = out_base + (uint32_t)(chunk_no % kGemmOutBufs) * kGemmOutBufBytes;
        // the store that last used this buffer must have finished reading it
        if (etid == 0) bulk_wait_group_read<kGemmOutBufs - 1>();
        if (etid == 0) { B200_TILE_TRACE(16 * min(job, 31) + 1 + 3 * (c / kGemmOutChunk)) }
        named_bar_sync(2, 128);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kSgmvBN + c + 32 * h), v);
          tmem_ld_wait();
          if (a.bias != nullptr) {
#pragma unroll
            for (int q = 0; q < 32; ++q) {
              const int cc = col0 + 32 * h + q;
              const float bv = cc < a.n_total ? __bfloat162float(a.bias[cc]) : 0.f;
              v[q] = __float_as_uint(__uint_as_float(v[q]) + bv);
            }
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[8 * q + 0]), __uint_as_float(v[8 * q + 1]));
            o.y = pack_bf16x2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]));
            o.z = pack_bf16x2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]));
            o.w = pack_bf16x2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]));
            if (neg_zero_row) o = make_uint4(0x80008000u, 0x80008000u, 0x80008000u, 0x80008000u);
            // 128-byte swizzle of the TMA box: 16-byte chunk index XOR (row % 8)
            const uint32_t chunk16 = (uint32_t)(4 * h + q) ^ (uint32_t)(row_in_blk & 7);
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(obuf + (uint32_t)row_in_blk * 128u + chunk16 * 16u),
                         "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w)
                         : "memory");
          }
        }
        if (etid == 0) { B200_TILE_TRACE(16 * min(job, 31) + 2 + 3 * (c / kGemmOutChunk)) }
        fence_proxy_async_smem();
        named_bar_sync(2, 128);
        if (etid == 0) { B200_TILE_TRACE(16 * min(job, 31) + 3 + 3 * (c / kGemmOutChunk)) }
        if (etid == 0) {
          if (a.expand_mode && !a.overwrite) tma_reduce_add_2d(&maps.y, obuf, col0, blk * kSgmvBM);
          else tma_store_2d_hint(&maps.y, obuf, col0, blk * kSgmvBM, l2_policy_evict_first());
          bulk_commit_group();
        }
      }
      tc_fence_before_sync();
      mbar_arrive(acc_empty(buf));
      if (etid == 0) { B200_TILE_TRACE(16 * min(job, 31) + 13) }
    }
    }
    if (etid == 0) bulk_wait_group_read<0>();
  }
  __syncthreads();
  B200_TILE_TRACE_CTA(1)
  if (warp == 1) tmem_dealloc(tmem_base, (uint32_t)tmem_cols);
  if (tid == 0 && abort_flag != 0) atomicOr(&g_b200_status, kStatusWaitGaveUp);
}

// ------------------------------------------------------------------ host side
inline size_t tc_tile_smem_bytes() { return (size_t)kGemmStages * kGemmStageBytes + kGemmOutBufs * kGemmOutBufBytes; }

// Slices must tile the packed output contiguously in 64-column units for the reduce path.
inline bool tc_expand_fast_path_ok(const SgmvArgs& a) {
  int pos = 0;
  for (int s = 0; s < a.n; ++s) {
    if (a.col[s] != pos || a.out[s] % kGemmOutChunk != 0) return false;
    pos += a.out[s];
  }
  return true;
}

// LoRA stages write D column ranges with an MMA N that is a multiple of 16.
inline bool tc_lora_stage_ok(const SgmvArgs& a) {
  for (int s = 0; s < a.n; ++s)
    if (a.col[s] % 16 != 0 || a.out[s] % 16 != 0) return false;
  return true;
}

// Tensor maps / arguments of tc_tile_kernel from the prefill kernels' (sgmv_prepare) ones.
// `weight` [n_total, in] row-major with pitch w_ld (LINEAR) or null (EXPAND).
inline int tc_tile_prepare(const SgmvMaps& sm, const SgmvArgs& sa, const void* weight, int64_t w_ld, int n_total,
                           const void* bias, bool expand_mode, bool lora, GemmMaps* maps, GemmArgs* args,
                           bool overwrite = false, bool after_shrink = true) {
  GemmArgs a = {};
  a.T = sa.T; a.in_dim = expand_mode ? 0 : sa.in_dim; a.n_total = n_total;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.S = sa.S; a.r_max = sa.r_max; a.n = sa.n;
  for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) { a.out[s] = sa.out[s]; a.col[s] = sa.col[s]; }
  a.token_to_slot = sa.token_to_slot;
  a.expand_mode = expand_mode ? 1 : 0;
  a.lora = lora ? 1 : 0;
  a.overwrite = overwrite ? 1 : 0;
  a.y = sa.y; a.y_ld = sa.y_ld;
  a.after_shrink = (lora && after_shrink) ? 1 : 0;  // the caller has just launched the shrink that writes tmp (else: unknown predecessor)
  maps->x = sm.x; maps->t = sm.t;
  for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) maps->b[s] = sm.b[s];
  maps->w = sm.x;
  if (!expand_mode) {
    if (int rc = make_tmap_2d(&maps->w, weight, (uint64_t)n_total, (uint64_t)sa.in_dim, (uint64_t)w_ld, kSgmvBN, kSgmvBK)) return rc;
  }
  if (int rc = make_tmap_2d(&maps->y, sa.y, (uint64_t)sa.T, (uint64_t)n_total, (uint64_t)sa.y_ld, kSgmvBM, kGemmOutChunk)) return rc;
  *args = a;
  return B200_LORA_OK;
}

inline int tc_tile_launch(const GemmMaps& maps, const GemmArgs& a, cudaStream_t stream) {
  const size_t smem = tc_tile_smem_bytes();
  if (a.S > 32767) return fail(B200_LORA_EUNSUPPORTED, "tile kernel: more than 32767 adapter slots");
  if (int rc = sgmv_set_smem(reinterpret_cast<const void*>(tc_tile_kernel), smem)) return rc;
  const int nblk = (a.T + kSgmvBM - 1) / kSgmvBM;
  const int ntile = (a.n_total + kSgmvBN - 1) / kSgmvBN;
  // One CTA per SM over equal contiguous tile ranges; more CTAs only when a range would otherwise
  // touch more than kTileMaxSeg row blocks (few column tiles per block and very many blocks).
  const int total = nblk * ntile;
  int ncta = std::min(kTileSMs, total);
  const int max_per = (kTileMaxSeg - 1) * ntile;
  if ((total + ncta - 1) / ncta > max_per) ncta = (total + max_per - 1) / max_per;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ncta, 1, 1);
  cfg.blockDim = dim3(kTileThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = bgmv_options().pdl ? 1 : 0;  // B200_LORA_OPT_PDL = 0: strict stream order
  cudaError_t e = cudaLaunchKernelEx(&cfg, tc_tile_kernel, maps, a);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(B200_LORA_ECUDA, "tc_tile_kernel launch: %s", cudaGetErrorString(e));
  }
  return B200_LORA_OK;
}

// y += LoRA delta for a prefill batch: shrink, then the reduce-add tile kernel (or the run-based
// expand when the slices do not tile the output in 64-column units).
// overwrite: y = delta (rows without adapter: -0.0) through plain tile stores, no read of y; only when the
// slices tile the output (prefill_overwrite_ok).
inline bool prefill_overwrite_ok(const SliceTable& st) {
  int pos = 0;
  for (int s = 0; s < st.n; ++s) {
    if (st.out[s] == 0) continue;
    if (st.col[s] != pos || st.out[s] % kGemmOutChunk != 0) return false;
    pos += st.out[s];
  }
  return pos > 0;
}

inline int prefill_add_launch(const SgmvProblem& b, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                              bool overwrite = false) {
  SgmvMaps sm;
  SgmvArgs sa;
  if (int rc = sgmv_prepare(b, workspace, workspace_bytes, &sm, &sa)) return rc;
  if (overwrite && !tc_expand_fast_path_ok(sa)) return fail(B200_LORA_EUNSUPPORTED, "prefill overwrite: slices do not tile the output");
  if (int rc = sgmv_launch_shrink(sm, sa, stream)) return rc;
  int n_total = 0;
  for (int s = 0; s < sa.n; ++s) n_total = std::max(n_total, sa.col[s] + sa.out[s]);
  if (tc_expand_fast_path_ok(sa)) {
    GemmMaps gm;
    GemmArgs ga;
    if (int rc = tc_tile_prepare(sm, sa, nullptr, 0, n_total, nullptr, true, true, &gm, &ga, overwrite)) return rc;
    return tc_tile_launch(gm, ga, stream);
  }
  return sgmv_launch_expand(sm, sa, stream);
}

struct LinearProblem {
  SgmvProblem lora;          // y, x, slabs, token_to_slot (null token_to_slot or no slice: plain linear)
  const void* weight; int64_t w_ld; int n_total; const void* bias;
};

// y = x . W^T (+ bias) + LoRA delta, the delta accumulated into the GEMM's TMEM accumulator.
inline int linear_lora_launch(const LinearProblem& p, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  const SgmvProblem& b = p.lora;
  if (b.in_dim % kSgmvBK != 0) return fail(B200_LORA_EUNSUPPORTED, "fused linear: in_dim must be a multiple of 64");
  if (p.n_total % 8 != 0 || p.w_ld % 8 != 0 || b.x_ld % 8 != 0 || b.y_ld % 8 != 0)
    return fail(B200_LORA_EUNSUPPORTED, "fused linear: widths and row strides must be multiples of 8");
  if ((reinterpret_cast<uintptr_t>(p.weight) & 15u) || (reinterpret_cast<uintptr_t>(b.x) & 15u) ||
      (reinterpret_cast<uintptr_t>(b.y) & 15u) || (reinterpret_cast<uintptr_t>(p.bias) & 1u))
    return fail(B200_LORA_EUNSUPPORTED, "fused linear: pointers must be 16-byte aligned");
  bool any = false;
  for (int s = 0; s < b.st.n; ++s) any = any || b.st.out[s] > 0;
  const bool with_lora = any && b.token_to_slot != nullptr;
  SgmvMaps sm;
  SgmvArgs sa = {};
  if (with_lora) {
    if (int rc = sgmv_prepare(b, workspace, workspace_bytes, &sm, &sa)) return rc;
    if (int rc = sgmv_launch_shrink(sm, sa, stream)) return rc;
  } else {
    // no adapter work: only the x and y views are needed
    sa.y = static_cast<__nv_bfloat16*>(b.y); sa.y_ld = b.y_ld; sa.T = b.T; sa.in_dim = b.in_dim; sa.S = 1; sa.r_max = 16;
    sa.n = 0; sa.token_to_slot = nullptr;
    if (int rc = make_tmap_2d(&sm.x, b.x, (uint64_t)b.T, (uint64_t)b.in_dim, (uint64_t)b.x_ld, kSgmvBM, kSgmvBK)) return rc;
    sm.t = sm.x;
    for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) { sm.a[s] = sm.x; sm.b[s] = sm.x; }
  }
  const bool fuse = with_lora && tc_lora_stage_ok(sa);
  GemmMaps gm;
  GemmArgs ga;
  if (int rc = tc_tile_prepare(sm, sa, p.weight, p.w_ld, p.n_total, p.bias, false, fuse, &gm, &ga)) return rc;
  if (int rc = tc_tile_launch(gm, ga, stream)) return rc;
  if (!with_lora || fuse) return B200_LORA_OK;
  return sgmv_launch_expand(sm, sa, stream);  // slices not 16-column aligned: delta in a second pass
}

}  // namespace b200lora
