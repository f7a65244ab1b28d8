// Fused decode multi-LoRA kernel (bf16): shrink + expand in ONE launch.
//
// Work decomposition
//   grid = (C, n_buckets), thread-block cluster = (C, 1, 1): one cluster per slot
//   bucket of the batch (bucket g = tokens sorted_idx[offsets[g] .. +counts[g]) that
//   all use adapter slot slot_ids[g]); buckets with id -1 or no tokens exit at once.
//   Inside a cluster the adapter's weights are split so that every byte of
//   lora_A[slot] and lora_B[slot] is pulled from HBM by exactly one CTA:
//     shrink : the n*r stacked rank rows are split across the C CTAs (full K each)
//     expand : each slice's output rows are split across the C CTAs
//   and the rank-r intermediate tmp[16 tokens, n*r] (bf16) is all-gathered through
//   distributed shared memory between the two phases (stores into every peer's buffer,
//   then one remote mbarrier arrive per peer; the buffer is double-buffered by pass).
//
// Roles
//   warp 8      producer: walks the CTA's tile list and issues 1-D bulk async copies
//               (cp.async.bulk, the TMA unit) into a ring of stages guarded by full/empty
//               mbarriers. A shrink tile is 8 rank rows x up to 1024 columns (one 16 KB
//               copy when the rows are contiguous, else 8 row copies), an expand tile is
//               one contiguous copy of up to 16 KB of lora_B rows. The weights do not
//               depend on the previous kernel of the stream, so under programmatic
//               dependent launch they are requested before griddepcontrol.wait.
//   warps 0-7   consumers: mma.sync m16n8k16 bf16 -> fp32 with tokens as the 16-row
//               operand (a pass handles 16 tokens of the bucket) and weight rows as the
//               8-column operand. Activations are read straight into MMA fragments
//               (16-byte global loads, once per 1024-column part); y is read one tile
//               ahead and written back with 16-byte stores.
//   Fragments are read as 16-byte vectors: thread (g,t) of a warp takes columns
//   [8t, 8t+8) of a 32-column block for both operands, which is a fixed permutation of the
//   k index shared by A and B and therefore leaves the dot products unchanged.
//
// Rows whose slot is -1 are in no bucket and are never read or written.
#pragma once

#include <cmath>
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace b200lora {

constexpr int kBgmvWarps = 8;                       // consumer warps
constexpr int kBgmvConsumers = kBgmvWarps * 32;
constexpr int kBgmvThreads = kBgmvConsumers + 32;   // + producer warp
constexpr int kBgmvTok = 16;           // tokens per pass (one MMA M tile)
constexpr int kBgmvMaxRc = 64;         // stacked rank rows per CTA
constexpr int kBgmvKP = 1024;          // columns per shrink tile
constexpr int kBgmvXBlocks = kBgmvKP / 32 / kBgmvWarps;  // 32-column blocks per warp and tile
constexpr int kBgmvSmemMax = 232448;   // 227 KB opt-in maximum per CTA
constexpr int kBgmvMaxStages = 12;
constexpr int kBgmvMaxExpandTiles = 256;  // expand tiles of one CTA (entries of its tile table)


// Optional phase timeline (SM clock) of rank-0 CTAs, compiled in only for tuning builds.
#ifdef B200_TRACE
__device__ long long g_b200_trace[1024 * 32];
#define B200_TRACE_AT(i, who) \
  if (tid == (who) && c == 0 && blockIdx.y < 1024) g_b200_trace[blockIdx.y * 32 + (i)] = clock64();
#else
#define B200_TRACE_AT(i, who)
#endif
#define B200_TRACE_POINT(i) B200_TRACE_AT(i, 0)
#define B200_TRACE_PRODUCER(i) B200_TRACE_AT(i, kBgmvConsumers)

struct BgmvProblem {
  void* y; int64_t y_ld; const void* x; int64_t x_ld;
  int T, in_dim, S, r_max;
  SliceTable st;
  const int32_t* rank_per_slot; const float* scale_per_slot;
  const int32_t *sorted_idx, *slot_ids, *counts, *offsets;
  int n_buckets; float scaling;
  // 0 = fused add; 1 = shrink only: tmp_io[s, t, 0:r] = scaling * x[t] . A_s[slot_t]^T (fp32, rows with an
  // adapter only); 2 = expand only: y += tmp_io . B^T. The pair serves the tensor-parallel exchange of tmp.
  // 3 = overwrite: y[t, cols] = delta for rows with an adapter and -0.0 for every other row (y is not
  // read); a base GEMM that then accumulates into y (beta = 1) gives base + delta, and x + (-0.0) == x
  // keeps rows without adapter bit-identical to the base result.
  int mode = 0;
  float* tmp_io = nullptr;  // [n_slices, T, r_max] fp32
  const int32_t* token_to_slot = nullptr;  // mode 3: which rows have no adapter
};

struct BgmvParams {
  __nv_bfloat16* y; int64_t y_ld; const __nv_bfloat16* x; int64_t x_ld;
  int T, in_dim, S, r_max;
  SliceTable st;  // active slices only
  const int32_t* rank_per_slot; const float* scale_per_slot;
  const int32_t *sorted_idx, *slot_ids, *counts, *offsets;
  int n_buckets; float scaling;
  int c_shift;      // cluster size C = 1 << c_shift
  int KP, nkp;      // columns per shrink tile (min(in, 1024)) and number of K parts
  int pitchA;       // bytes between rows of a shrink tile (KP*2, +64 when rows are copied one by one)
  int ER, er_shift; // out rows per expand tile (power of two, 32..256)
  int oc[B200_LORA_MAX_SLICES];  // out rows of each slice owned by one CTA (multiple of 32)
  int stage_bytes, NS;
  int red_pitch;    // floats per token row of the cross-warp reduction buffer
  int pitchT;       // bytes per token row of tmp
  int tmp_bytes;    // bytes of one tmp buffer
  int off_red, off_tmp, off_tab, off_bar;
  int full_k;       // every K part has all 1024 columns
  int y_cols;       // columns of y that the slices may touch (largest column end)
  int ksplit;       // 1: the K parts (not the rank rows) are dealt over the CTAs of a cluster
  int pitchR, recv_bytes, off_recv;  // K split: floats per token row / bytes of one buffer of received partial sums
  int use_pdl;
  int mode;         // 0 fused, 1 shrink only (tmp_io written), 2 expand only (tmp_io read), 3 overwrite y
  float* tmp_io;
  const int32_t* token_to_slot;
};

__host__ __device__ __forceinline__ int ceil_div_i(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ __forceinline__ int round_up_i(int a, int b) { return ceil_div_i(a, b) * b; }

// mode 3: rows that get no delta (no adapter, unknown slot, adapter of rank 0) are set to -0.0 over the
// columns of all slices; the rows are dealt over the CTAs of the grid, `nthreads` threads of each taking part.
__device__ __forceinline__ void bgmv_fill_rows_without_delta(const BgmvParams& p, int cta, int n_ctas, int thread, int nthreads) {
  const uint4 negz = make_uint4(0x80008000u, 0x80008000u, 0x80008000u, 0x80008000u);
  for (int row = cta; row < p.T; row += n_ctas) {
    const int sl = p.token_to_slot[row];
    bool dead = sl < 0 || sl >= p.S;
    if (!dead && p.rank_per_slot != nullptr) dead = p.rank_per_slot[sl] <= 0;
    if (!dead) continue;
#pragma unroll
    for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) {
      if (s < p.st.n) {
        __nv_bfloat16* dst = p.y + (int64_t)row * p.y_ld + p.st.col[s];
        for (int i = thread; i < (p.st.out[s] >> 3); i += nthreads) stg128(dst + 8 * i, negz);
      }
    }
  }
}

// Two CTAs per SM: the CTAs of the next launch of the stream become resident while this launch still
// runs, so their weight copies and L2 prefetches overlap this launch's dependent chain.
#ifndef BGMV_MINBLOCKS
#define BGMV_MINBLOCKS 2
#endif
// kMode = BgmvParams::mode, compiled separately so that no path carries the branches of another;
// kFullK = every K part has all 1024 columns (in_dim a multiple of 1024): no column checks in the shrink
template <int kMode, bool kFullK>
__global__ void __launch_bounds__(kBgmvThreads, BGMV_MINBLOCKS) bgmv_fused_kernel(const __grid_constant__ BgmvParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int bucket = blockIdx.y;
  const int C = 1 << p.c_shift;
  const int c = (int)cluster_ctarank();
  const int NS = p.NS;
  constexpr bool kOverwrite = kMode == 3;
  constexpr int mode = kMode;

  B200_TRACE_POINT(0)
  // Let the next launch of the stream start at once: before its own griddepcontrol.wait it only
  // reads index metadata and lora slabs, which no kernel of this library writes, so its weight
  // traffic overlaps this kernel's compute and keeps HBM busy across launch boundaries.
  if (p.use_pdl) griddep_launch_dependents();
  // ---- bucket metadata (uniform across the cluster); barrier set-up overlaps the loads
  const int slot = p.slot_ids[bucket];
  const int cnt = p.counts[bucket];
  const int start = p.offsets[bucket];

  float* red = reinterpret_cast<float*>(smem + p.off_red);
  uint8_t* tmp_base = smem + p.off_tmp;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.off_bar);  // full[], empty[], tmp_ready[2]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * kBgmvMaxStages + 2);
  const uint32_t bar_base = smem_u32(bars);
  const uint32_t ring_base = smem_u32(smem);
  // one barrier per tmp buffer: pass p uses barrier p & 1 in phase (p >> 1) & 1
  const uint32_t tmp_ready_bars = bar_base + 8u * (uint32_t)(2 * kBgmvMaxStages);
  auto full_bar = [&](int s) { return bar_base + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (uint32_t)(kBgmvMaxStages + s); };
  if (tid < NS) {
    mbar_init(full_bar(tid), 1);
    mbar_init(empty_bar(tid), kBgmvWarps);
    if (tid == 0) {
      mbar_init(tmp_ready_bars, 1u);  // completed by byte count (st.async from every CTA of the cluster)
      mbar_init(tmp_ready_bars + 8u, 1u);
      *abort_flag = 0;
    }
    mbar_fence_init();
  }

  int rank = p.r_max;
  if (p.rank_per_slot != nullptr && slot >= 0 && slot < p.S) rank = min(max(p.rank_per_slot[slot], 0), p.r_max);
  const int r_eff = min(p.r_max, (rank + 31) & ~31);
  // (a bucket whose row range leaves the batch is ignored; the bounds-checked build reports it)
  if (cnt > 0 && slot >= 0) (void)B200_IN_BOUNDS(slot < p.S && start >= 0 && start <= p.T - cnt);
  if (slot < 0 || slot >= p.S || cnt <= 0 || start < 0 || start > p.T - cnt || r_eff == 0) {
    // An idle cluster holds nothing, but one CTA of every launch must outlive the previous launch
    // of the stream: a launch that ended before its predecessor would let the launch behind it
    // pass its own wait too early.
    if (p.use_pdl && (kOverwrite || (bucket == 0 && c == 0))) griddep_wait();
    if (kOverwrite)  // an idle cluster still does its share of the -0.0 rows
      bgmv_fill_rows_without_delta(p, bucket * C + c, (int)gridDim.y * C, tid, kBgmvThreads);
    return;
  }
  const float sc = p.scaling * (p.scale_per_slot != nullptr ? p.scale_per_slot[slot] : 1.0f);
  B200_TRACE_POINT(1)

  const int n = p.st.n;
  const int in_dim = p.in_dim;
  const int Q = n * r_eff;                                       // stacked rank rows
  // Shrink work of the cluster: either the rank rows are split over the CTAs (each takes all K parts of
  // its rows, the bf16 results are all-gathered), or - long input rows - the K parts are dealt over the
  // CTAs (each takes all rank rows of its K parts, the fp32 partial sums are exchanged and added).
  const bool ksplit = (kMode == 0 || kMode == 3) && p.ksplit != 0;
  const int Rc = ksplit ? Q : ((((Q + C - 1) >> p.c_shift) + 7) & ~7);  // rows owned per CTA
  const int q_lo = ksplit ? 0 : min(c * Rc, Q);
  const int rows_c = mode == 2 ? 0 : min(q_lo + Rc, Q) - q_lo;   // multiple of 8, may be 0 (expand only: no shrink rows)
  const int nt_c = rows_c >> 3;                                  // 8-row tiles of this CTA
  const int KP = p.KP, pitchA = p.pitchA, ER = p.ER, nkp = p.nkp;
  const int kp0 = ksplit ? c : 0, kstep = ksplit ? C : 1;        // K parts of this CTA: kp0, kp0 + kstep, ...
  const int nkp_c = ksplit ? (nkp > c ? (nkp - c + C - 1) >> p.c_shift : 0) : nkp;
  const int shrink_tiles = nt_c * nkp_c;
  int e_lo[B200_LORA_MAX_SLICES], e_n[B200_LORA_MAX_SLICES], e_tiles[B200_LORA_MAX_SLICES];
  int tiles_exp = 0;
#pragma unroll
  for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) {
    e_lo[s] = e_n[s] = e_tiles[s] = 0;
    if (s < n && mode != 1) {  // (shrink only: no expand tiles)
      const int out = p.st.out[s];
      e_lo[s] = min(c * p.oc[s], out);
      e_n[s] = min(e_lo[s] + p.oc[s], out) - e_lo[s];
      e_tiles[s] = (e_n[s] + ER - 1) >> p.er_shift;
      tiles_exp += e_tiles[s];
    }
  }
  const int npass = (cnt + kBgmvTok - 1) >> 4;
  const int total = (shrink_tiles + tiles_exp) * npass;
  // bytes a pass delivers into this CTA: 16 token rows of all Q stacked rank rows, as bf16 once
  // (all-gather) or as fp32 from every CTA of the cluster (K split)
  const uint32_t gather_bytes = ksplit ? (uint32_t)(C * kBgmvTok * Q * 4) : (uint32_t)(kBgmvTok * Q * 2);
  if (tid == 0 && (mode == 0 || mode == 3)) {
    mbar_arrive_expect_tx(tmp_ready_bars, gather_bytes);                      // pass 0
    if (npass > 1) mbar_arrive_expect_tx(tmp_ready_bars + 8u, gather_bytes);  // pass 1
  }

  __syncthreads();  // barriers initialised
  B200_TRACE_POINT(2)
  // Start-up cluster barrier: every CTA of the cluster has initialised its barriers once it
  // completes. Consumers wait on it before their first remote store, the producer before it exits.
  cluster_arrive();

  if (warp == kBgmvWarps) {
    // =========================== producer warp ===========================
    int i_shrink = shrink_tiles > 0 ? 1 : 0, i_kp = 0, i_j = 0;  // cursor: phase, K part, 8-row tile
    int i_s = 0, i_et = 0;                                       // cursor: slice / tile in slice
    int i_qs = 0, i_qr = q_lo;                                   // slice / row of the cursor's first rank row
    while (i_qr >= r_eff) { i_qr -= r_eff; ++i_qs; }
    const int q0_s = i_qs, q0_r = i_qr;
    int p_stage = 0, p_round = 0;
    const int npro = min(NS, total);
#pragma unroll 1
    for (int it = 0; it < total; ++it) {
      if (p_round > 0) mbar_wait_bounded(empty_bar(p_stage), (uint32_t)((p_round & 1) ^ 1), abort_flag);
      const uint32_t sbase = ring_base + (uint32_t)p_stage * (uint32_t)p.stage_bytes;
      const uint32_t fb = full_bar(p_stage);
      if (i_shrink) {
        const int k0 = (kp0 + i_kp * kstep) * KP;
        const uint32_t row_bytes = (uint32_t)min(KP, in_dim - k0) * 2u;
        const void* aptr = nullptr;
#pragma unroll
        for (int s = 0; s < B200_LORA_MAX_SLICES; ++s)
          if (s == i_qs) aptr = p.st.a[s];
        const __nv_bfloat16* src =
            static_cast<const __nv_bfloat16*>(aptr) + ((int64_t)slot * p.r_max + i_qr) * in_dim + k0;
        // 8 rank rows of slice i_qs, columns [k0, k0 + row_bytes / 2), into stage p_stage
        if (!B200_IN_BOUNDS(aptr != nullptr && i_qs < n && i_qr + 8 <= p.r_max && k0 < in_dim && p_stage < NS &&
                            8 * pitchA <= p.stage_bytes)) {
          if (lane == 0) mbar_arrive(fb);  // the tile is skipped; its consumers see stale bytes, never a stuck barrier
        } else
        if (nkp == 1) {
          // the 8 rows are contiguous in the slab: one copy (each copy costs the TMA unit ~100 cycles)
          if (lane == 0) {
            mbar_arrive_expect_tx(fb, 8u * row_bytes);
            bulk_g2s(sbase, src, 8u * row_bytes, fb);
          }
        } else {
          if (lane == 0) mbar_arrive_expect_tx(fb, 8u * row_bytes);
          __syncwarp();
          if (lane < 8) bulk_g2s(sbase + (uint32_t)(lane * pitchA), src + (int64_t)lane * in_dim, row_bytes, fb);
        }
        // advance: 8-row tiles inner, K parts outer
        ++i_j;
        i_qr += 8;
        if (i_qr >= r_eff) { i_qr = 0; ++i_qs; }
        if (i_j == nt_c) {
          i_j = 0; i_qs = q0_s; i_qr = q0_r;
          // (shrink-only launches have no expand tiles: the next pass starts with shrink tiles again)
          if (++i_kp == nkp_c) { i_kp = 0; i_shrink = tiles_exp > 0 ? 0 : 1; i_s = 0; i_et = 0; }
        }
      } else {
#pragma unroll
        for (int s = 0; s < B200_LORA_MAX_SLICES - 1; ++s)  // skip slices this CTA has no tiles of
          if (i_s == s && i_et >= e_tiles[s]) { i_s = s + 1; i_et = 0; }
        int lo = 0, en = 0, out = 0, left = 0;
        const void* bptr = nullptr;
#pragma unroll
        for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) {
          if (s == i_s) { lo = e_lo[s]; en = e_n[s]; out = p.st.out[s]; bptr = p.st.b[s]; left = e_tiles[s]; }
          if (s > i_s) left += e_tiles[s];
        }
        const int r0 = i_et << p.er_shift;
        const int nrows = min(ER, en - r0);
        if (!B200_IN_BOUNDS(bptr != nullptr && nrows > 0 && lo + r0 + nrows <= out && p_stage < NS &&
                            nrows * p.r_max * 2 <= p.stage_bytes)) {
          if (lane == 0) mbar_arrive(fb);
        } else
        if (lane == 0) {
          const uint32_t bytes = (uint32_t)nrows * (uint32_t)p.r_max * 2u;
          mbar_arrive_expect_tx(fb, bytes);
          const __nv_bfloat16* src =
              static_cast<const __nv_bfloat16*>(bptr) + ((int64_t)slot * out + lo + r0) * p.r_max;
          bulk_g2s(sbase, src, bytes, fb);
        }
        ++i_et;
        // `left` = tiles of this and later slices; after the last one the next pass starts
        // with its shrink tiles again
        if (i_et >= left) {
          i_shrink = shrink_tiles > 0 ? 1 : 0;
          i_kp = 0; i_j = 0; i_qs = q0_s; i_qr = q0_r; i_s = 0; i_et = 0;
        }
      }
      __syncwarp();
      if (++p_stage == NS) { p_stage = 0; ++p_round; }
      if (it + 1 == npro) {
        B200_TRACE_PRODUCER(3)
        // The ring is full and the previous launch of the stream may still be running: ask the L2 for
        // the rest of this CTA's weights now, so that the refills that follow the wait find them there.
        if (shrink_tiles + tiles_exp > npro && ksplit) {
          // one row piece per lane: rank row q of this CTA's K part ikp
#pragma unroll 1
          for (int idx = lane; idx < rows_c * nkp_c; idx += 32) {
            const int ikp = idx / max(rows_c, 1), q = idx - ikp * rows_c;
            const int s = q / r_eff, r0 = q - s * r_eff, k0 = (kp0 + ikp * kstep) * KP;
            const void* aptr = nullptr;
#pragma unroll
            for (int ss = 0; ss < B200_LORA_MAX_SLICES; ++ss)
              if (ss == s) aptr = p.st.a[ss];
            bulk_prefetch_l2(static_cast<const __nv_bfloat16*>(aptr) + ((int64_t)slot * p.r_max + r0) * in_dim + k0,
                             (uint32_t)min(KP, in_dim - k0) * 2u);
          }
        }
        if (shrink_tiles + tiles_exp > npro && lane == 0) {
          int q = q_lo;
          const int q_hi = ksplit ? q_lo : q_lo + rows_c;
#pragma unroll 1
          while (q < q_hi) {
            const int s = q / r_eff, r0 = q - s * r_eff;
            const int nr = min(r_eff - r0, q_hi - q);
            const void* aptr = nullptr;
#pragma unroll
            for (int ss = 0; ss < B200_LORA_MAX_SLICES; ++ss)
              if (ss == s) aptr = p.st.a[ss];
            bulk_prefetch_l2(static_cast<const __nv_bfloat16*>(aptr) + ((int64_t)slot * p.r_max + r0) * in_dim,
                             (uint32_t)nr * (uint32_t)in_dim * 2u);
            q += nr;
          }
#pragma unroll
          for (int s = 0; s < B200_LORA_MAX_SLICES; ++s)
            if (s < n && e_n[s] > 0)
              bulk_prefetch_l2(static_cast<const __nv_bfloat16*>(p.st.b[s]) + ((int64_t)slot * p.st.out[s] + e_lo[s]) * p.r_max,
                               (uint32_t)e_n[s] * (uint32_t)p.r_max * 2u);
        }
      }
    }
    cluster_wait();
    return;
  }

  // ============================= consumer warps =============================
  // Everything that does not depend on the previous launch of the stream is done before the wait:
  // token rows, the table of this CTA's expand tiles, thread-constant address pieces and L2 prefetches
  // (a prefetch never creates stale data: L2 is the point of coherence). What runs after the wait is
  // the dependent chain activations -> shrink -> all-gather -> expand, kept as short as possible.
  int tok0_lo = -1, tok0_hi = -1;
  if (g < cnt) tok0_lo = p.sorted_idx[start + g];
  if (g + 8 < cnt) tok0_hi = p.sorted_idx[start + g + 8];
  (void)B200_IN_BOUNDS(tok0_lo < p.T && tok0_hi < p.T && tok0_lo >= -1 && tok0_hi >= -1);
  if (tok0_lo >= p.T) tok0_lo = -1;
  if (tok0_hi >= p.T) tok0_hi = -1;

  // expand tile e of this CTA (ring order): x = first y column, y = rows | slice << 16
  int2* etab = reinterpret_cast<int2*>(smem + p.off_tab);
#pragma unroll 1
  for (int e = tid; e < tiles_exp; e += kBgmvConsumers) {
    int s_e = 0, et = e;
#pragma unroll
    for (int s = 0; s < B200_LORA_MAX_SLICES - 1; ++s)
      if (s_e == s && et >= e_tiles[s]) { et -= e_tiles[s]; s_e = s + 1; }
    int lo = 0, en = 0, cb = 0;
#pragma unroll
    for (int s = 0; s < B200_LORA_MAX_SLICES; ++s)
      if (s == s_e) { lo = e_lo[s]; en = e_n[s]; cb = p.st.col[s]; }
    const int r0 = et << p.er_shift;
    etab[e] = make_int2(cb + lo + r0, min(ER, en - r0) | (s_e << 16));
  }
  named_bar_sync(1, kBgmvConsumers);  // table complete

  const int rb = warp * 32;             // expand: out rows of this warp inside a tile
  const int x_col = warp * 32 + t * 8;  // shrink: first column of the thread inside a K part (block i adds 256)
  const int y_col = rb + 8 * t;         // expand: first of the thread's 8 output columns inside a tile
  if (p.use_pdl) {
#pragma unroll 1
    for (int ikp = 0; ikp < (rows_c > 0 ? nkp_c : 0); ++ikp) {
      const int k0 = (kp0 + ikp * kstep) * KP;
#pragma unroll 1
      for (int kc = k0 + x_col; kc < min(k0 + KP, in_dim); kc += kBgmvWarps * 32) {
        if (tok0_lo >= 0) prefetch_l2(p.x + (int64_t)tok0_lo * p.x_ld + kc);
        if (tok0_hi >= 0) prefetch_l2(p.x + (int64_t)tok0_hi * p.x_ld + kc);
      }
    }
    if (!kOverwrite) {  // the lines of y that this thread's reductions will land in
#pragma unroll 1
      for (int e = 0; e < tiles_exp; ++e) {
        const int2 te = etab[e];
        if (y_col < (te.y & 0xffff)) {
          if (tok0_lo >= 0) prefetch_l2(p.y + (int64_t)tok0_lo * p.y_ld + te.x + y_col);
          if (tok0_hi >= 0) prefetch_l2(p.y + (int64_t)tok0_hi * p.y_ld + te.x + y_col);
        }
      }
    }
  }

  // thread-constant pieces of the shared-memory addresses
  const uint32_t pitchB = (uint32_t)p.r_max * 2u;
  const uint32_t a_off = (uint32_t)(g * pitchA + x_col * 2);                            // shrink tile: row g
  const uint32_t w_off = (uint32_t)(rb + 8 * (g >> 1) + (g & 1)) * pitchB + (uint32_t)t * 16u;  // expand tile
  // MMA column n of n-tile j reads slab row 8*(n/2) + 2j + (n%2) of the warp's 32 rows: thread (g,t)
  // then owns 8 consecutive output columns 8t..8t+7 of the block.
  const uint32_t t_off = (uint32_t)(g * p.pitchT + t * 16);                             // tmp: token row g
  float* const red_wr = red + ((size_t)warp * kBgmvTok + g) * p.red_pitch + 2 * t;      // + 8 * pitch: token g + 8
  const int kblocks = r_eff >> 5;
  // all-gather item of this thread: one token row x four consecutive rank rows of this CTA
  const int groups = rows_c >> 2;
  const bool has_item = tid < kBgmvTok * groups;
  const int it_tok = has_item ? tid / max(groups, 1) : 0;
  const int it_q = q_lo + 4 * (has_item ? tid - it_tok * groups : 0);
  const float* const red_rd = red + (size_t)it_tok * p.red_pitch + (it_q - q_lo);
  const uint32_t it_off = (uint32_t)(it_tok * p.pitchT + it_q * 2);
  const uint32_t tmp_u32 = smem_u32(tmp_base);
  const uint32_t recv_u32 = smem_u32(smem + p.off_recv);
  const uint32_t it_roff = (uint32_t)(it_tok * p.pitchR + it_q) * 4u;  // K split: the item inside one sender's block

  if (p.use_pdl) griddep_wait();  // x and y of this launch are final from here on
  if (kOverwrite) bgmv_fill_rows_without_delta(p, bucket * C + c, (int)gridDim.y * C, tid, kBgmvConsumers);
  B200_TRACE_POINT(4)

  int c_stage = 0;
  uint32_t c_parity = 0, stage_addr = ring_base;  // stage being consumed: index, phase, address
  auto advance = [&]() {
    stage_addr += (uint32_t)p.stage_bytes;
    if (++c_stage == NS) { c_stage = 0; c_parity ^= 1u; stage_addr = ring_base; }
  };

#pragma unroll 1
  for (int pass = 0; pass < npass; ++pass) {
    int tok_lo = tok0_lo, tok_hi = tok0_hi;
    if (pass > 0) {
      tok_lo = tok_hi = -1;
      if (pass * kBgmvTok + g < cnt) tok_lo = p.sorted_idx[start + pass * kBgmvTok + g];
      if (pass * kBgmvTok + g + 8 < cnt) tok_hi = p.sorted_idx[start + pass * kBgmvTok + g + 8];
      (void)B200_IN_BOUNDS(tok_lo < p.T && tok_hi < p.T && tok_lo >= -1 && tok_hi >= -1);
      if (tok_lo >= p.T) tok_lo = -1;
      if (tok_hi >= p.T) tok_hi = -1;
    }
    const __nv_bfloat16* const xlo_p = p.x + (int64_t)max(tok_lo, 0) * p.x_ld + x_col;
    const __nv_bfloat16* const xhi_p = p.x + (int64_t)max(tok_hi, 0) * p.x_ld + x_col;
    __nv_bfloat16* const ylo_p = p.y + (int64_t)max(tok_lo, 0) * p.y_ld + y_col;
    __nv_bfloat16* const yhi_p = p.y + (int64_t)max(tok_hi, 0) * p.y_ld + y_col;

    // ===== shrink: red[warp][tok][row] = x[16 tok, K blocks of this warp] . A_rows^T =====
#pragma unroll 1
    for (int kp = 0; kp < (rows_c > 0 ? nkp_c : 0); ++kp) {
      const int k0 = (kp0 + kp * kstep) * KP;
      // activation fragments of this warp's 32-column blocks, kept for all row tiles
      uint4 xlo[kBgmvXBlocks], xhi[kBgmvXBlocks];
#pragma unroll
      for (int i = 0; i < kBgmvXBlocks; ++i) {
        xlo[i] = xhi[i] = make_uint4(0, 0, 0, 0);
        if (kFullK || (x_col + 256 * i < KP && k0 + x_col + 256 * i < in_dim)) {
          if (tok_lo >= 0) xlo[i] = ldg128_nc(xlo_p + k0 + 256 * i);
          if (tok_hi >= 0) xhi[i] = ldg128_nc(xhi_p + k0 + 256 * i);
        }
      }
      // kTiles (1 or 2) 8-row tiles of the ring against the warp's activation fragments: all loads
      // first, then the independent MMA chains of both tiles, then the stores; sums of the K blocks go
      // to the warp's rows of the reduction buffer (added to what earlier K parts left there)
      auto shrink_tiles_fn = [&](auto n_tiles, int j, uint32_t addr0, uint32_t addr1) {
        constexpr int kTiles = decltype(n_tiles)::value;
        float acc[kTiles][2][4];
#pragma unroll
        for (int u = 0; u < kTiles; ++u)
#pragma unroll
          for (int h = 0; h < 2; ++h) acc[u][h][0] = acc[u][h][1] = acc[u][h][2] = acc[u][h][3] = 0.f;
#pragma unroll
        for (int i = 0; i < kBgmvXBlocks; ++i) {
          uint4 w[kTiles];
#pragma unroll
          for (int u = 0; u < kTiles; ++u) {
            w[u] = make_uint4(0, 0, 0, 0);
            if (kFullK || (x_col + 256 * i < KP && k0 + x_col + 256 * i < in_dim))
              w[u] = lds128((u == 0 ? addr0 : addr1) + a_off + 512u * i);
          }
#pragma unroll
          for (int u = 0; u < kTiles; ++u) {
            mma_bf16_16816(acc[u][0], xlo[i].x, xhi[i].x, xlo[i].y, xhi[i].y, w[u].x, w[u].y);
            mma_bf16_16816(acc[u][1], xlo[i].z, xhi[i].z, xlo[i].w, xhi[i].w, w[u].z, w[u].w);
          }
        }
#pragma unroll
        for (int u = 0; u < kTiles; ++u) {
          // acc holds (tok g | g+8, rank rows 8(j+u)+2t, 8(j+u)+2t+1)
          float2* r0 = reinterpret_cast<float2*>(red_wr + 8 * (j + u));
          float2* r1 = reinterpret_cast<float2*>(red_wr + 8 * p.red_pitch + 8 * (j + u));
          float2 a = make_float2(0.f, 0.f), b = a;
          if (kp != 0) { a = *r0; b = *r1; }
          *r0 = make_float2(a.x + acc[u][0][0] + acc[u][1][0], a.y + acc[u][0][1] + acc[u][1][1]);
          *r1 = make_float2(b.x + acc[u][0][2] + acc[u][1][2], b.y + acc[u][0][3] + acc[u][1][3]);
        }
      };
      int j = 0;
#pragma unroll 1
      for (; j + 1 < nt_c; j += 2) {
        const int s0 = c_stage;
        const uint32_t a0 = stage_addr;
        mbar_wait_bounded(full_bar(s0), c_parity, abort_flag);
        if (kp == 0 && j == 0 && pass == 0) { B200_TRACE_POINT(5) }
        advance();
        const int s1 = c_stage;
        const uint32_t a1 = stage_addr;
        mbar_wait_bounded(full_bar(s1), c_parity, abort_flag);
        advance();
        shrink_tiles_fn(std::integral_constant<int, 2>{}, j, a0, a1);
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_relaxed(empty_bar(s0));
          mbar_arrive_relaxed(empty_bar(s1));
        }
      }
#pragma unroll 1
      for (; j < nt_c; ++j) {
        mbar_wait_bounded(full_bar(c_stage), c_parity, abort_flag);
        if (kp == 0 && j == 0 && pass == 0) { B200_TRACE_POINT(5) }
        shrink_tiles_fn(std::integral_constant<int, 1>{}, j, stage_addr, stage_addr);
        __syncwarp();
        if (lane == 0) mbar_arrive_relaxed(empty_bar(c_stage));
        advance();
      }
    }
    if (pass == 0) { B200_TRACE_POINT(6) }

    // ===== cross-warp reduction of the K slices, scale, bf16, all-gather =====
    // the barrier of pass + 1 is armed one pass ahead (passes 0 and 1 at start-up): every local wait on
    // its previous phase is over, and no peer sends for pass + 1 before it has this pass from this CTA
    if (tid == 0 && pass >= 1 && pass + 1 < npass && (mode == 0 || mode == 3))
      mbar_arrive_expect_tx(tmp_ready_bars + 8u * (uint32_t)((pass + 1) & 1), gather_bytes);
    named_bar_sync(1, kBgmvConsumers);
    if (pass == 0) {
      B200_TRACE_POINT(7)
      cluster_wait();  // start-up barrier: peers run and their barriers are initialised
    }
    const uint32_t tmp_cur = tmp_u32 + (uint32_t)((pass & 1) * p.tmp_bytes);
    const uint32_t tmp_ready_bar = tmp_ready_bars + 8u * (uint32_t)(pass & 1);
    if (mode == 2) {
      // expand only: tmp of this pass comes from global memory (fp32 [n, T, r_max], summed over the
      // tensor-parallel ranks) and is rounded to bf16 into this CTA's own buffer
      uint8_t* tmp_full = tmp_base + (size_t)(pass & 1) * p.tmp_bytes;
      const int tok = tid >> 4;
      int trow = -1;
      if (pass * kBgmvTok + tok < cnt) trow = p.sorted_idx[start + pass * kBgmvTok + tok];
      if (trow >= p.T) trow = -1;
#pragma unroll 1
      for (int pr = tid & 15; pr < (Q >> 1); pr += 16) {
        const int q = 2 * pr, s = q / r_eff, rr = q - s * r_eff;
        float2 v = make_float2(0.f, 0.f);
        if (trow >= 0) v = *reinterpret_cast<const float2*>(p.tmp_io + ((int64_t)s * p.T + trow) * p.r_max + rr);
        *reinterpret_cast<uint32_t*>(tmp_full + (size_t)tok * p.pitchT + (size_t)q * 2) = pack_bf16x2(v.x, v.y);
      }
      named_bar_sync(1, kBgmvConsumers);
    } else {
      if (has_item) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < kBgmvWarps; ++w) {
          const float4 v = *reinterpret_cast<const float4*>(red_rd + (size_t)w * kBgmvTok * p.red_pitch);
          a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
        if (mode == 1) {
          // shrink only: fp32 result of this CTA's rank rows straight to global memory
          int trow = -1;
          if (pass * kBgmvTok + it_tok < cnt) trow = p.sorted_idx[start + pass * kBgmvTok + it_tok];
          if (trow >= 0 && trow < p.T) {
            const int s = it_q / r_eff, rr = it_q - s * r_eff;
            float2* dst = reinterpret_cast<float2*>(p.tmp_io + ((int64_t)s * p.T + trow) * p.r_max + rr);
            dst[0] = make_float2(a.x * sc, a.y * sc);
            dst[1] = make_float2(a.z * sc, a.w * sc);
          }
        } else if (ksplit) {
          // to every CTA of the cluster (this one included): this CTA's fp32 partial sums over its K parts,
          // into the block the receiver keeps for this sender
          const uint32_t dst = recv_u32 + (uint32_t)(((pass & 1) * C + c) * (kBgmvTok * p.pitchR * 4)) + it_roff;
#pragma unroll 1
          for (int rc = 0; rc < C; ++rc)
            st_async_f32x4(mapa_shared(dst, (uint32_t)rc), a, mapa_shared(tmp_ready_bar, (uint32_t)rc));
        } else {
          // to every CTA of the cluster (this one included): 8 bytes of tmp + their count on the
          // receiver's barrier in one operation
          const uint32_t v0 = pack_bf16x2(a.x * sc, a.y * sc), v1 = pack_bf16x2(a.z * sc, a.w * sc);
#pragma unroll 1
          for (int rc = 0; rc < C; ++rc)
            st_async_b32x2(mapa_shared(tmp_cur + it_off, (uint32_t)rc), v0, v1, mapa_shared(tmp_ready_bar, (uint32_t)rc));
        }
      }
      if (mode == 1) {
        named_bar_sync(1, kBgmvConsumers);  // all warps have read the reduction buffer before the next pass refills it
        continue;
      }
      if (pass == 0) { B200_TRACE_POINT(8) }
      // (the wait also orders the reduction buffer: no warp passes it before every warp of every CTA
      // of the cluster has summed and sent its items, so the next pass may refill the buffer)
      mbar_wait_bounded_acquire_cluster(tmp_ready_bar, (uint32_t)((pass >> 1) & 1), abort_flag);
      if (ksplit) {
        // add the C partial sums of this thread's item, scale, round: tmp of this pass, kept locally
        if (has_item) {
          float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
          const float* src = reinterpret_cast<const float*>(smem + p.off_recv) + (size_t)(pass & 1) * C * kBgmvTok * p.pitchR +
                             (size_t)it_tok * p.pitchR + it_q;
#pragma unroll 1
          for (int rc = 0; rc < C; ++rc) {
            const float4 v = *reinterpret_cast<const float4*>(src + (size_t)rc * kBgmvTok * p.pitchR);
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
          }
          *reinterpret_cast<uint2*>(tmp_base + (size_t)(pass & 1) * p.tmp_bytes + it_off) =
              make_uint2(pack_bf16x2(a.x * sc, a.y * sc), pack_bf16x2(a.z * sc, a.w * sc));
        }
        named_bar_sync(1, kBgmvConsumers);
      }
      if (pass == 0) { B200_TRACE_POINT(9) }
    }

    // ===== expand: y[tok, cols] += tmp[16 tok, r] . B_rows^T ======================
    // one tile of the ring per step: one 32-row block per warp (ER <= 256). Rows of a stage beyond the
    // tile's rows hold stale bytes; their products land in columns that are not written.
    auto expand_fn = [&](int e, uint32_t tile_addr) {
      const int2 te = etab[e];
      float d[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) d[j][0] = d[j][1] = d[j][2] = d[j][3] = 0.f;
      const uint32_t a_addr = tmp_cur + t_off + (uint32_t)((te.y >> 16) * r_eff * 2);
      const uint32_t w_addr = tile_addr + w_off;
#pragma unroll 1
      for (int kb = 0; kb < kblocks; ++kb) {
        const uint4 alo = lds128(a_addr + 64u * kb);
        const uint4 ahi = lds128(a_addr + 64u * kb + 8u * (uint32_t)p.pitchT);
        uint4 w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = lds128(w_addr + 64u * kb + 2u * j * pitchB);
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16_16816(d[j], alo.x, ahi.x, alo.y, ahi.y, w[j].x, w[j].y);
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16_16816(d[j], alo.z, ahi.z, alo.w, ahi.w, w[j].z, w[j].w);
      }
      if (y_col < (te.y & 0xffff) && B200_IN_BOUNDS(te.x >= 0 && te.x + y_col + 8 <= p.y_cols)) {
        const uint4 lo4 = make_uint4(pack_bf16x2(d[0][0], d[0][1]), pack_bf16x2(d[1][0], d[1][1]),
                                     pack_bf16x2(d[2][0], d[2][1]), pack_bf16x2(d[3][0], d[3][1]));
        const uint4 hi4 = make_uint4(pack_bf16x2(d[0][2], d[0][3]), pack_bf16x2(d[1][2], d[1][3]),
                                     pack_bf16x2(d[2][2], d[2][3]), pack_bf16x2(d[3][2], d[3][3]));
        if (kOverwrite) {
          if (tok_lo >= 0) stg128(ylo_p + te.x, lo4);
          if (tok_hi >= 0) stg128(yhi_p + te.x, hi4);
        } else {
          // The delta is rounded to bf16 and added to y by one 16-byte reduction at the L2: y never
          // travels to the SM and nothing waits for it. Each element of y receives exactly one
          // reduction per launch, so the result does not depend on their order.
          if (tok_lo >= 0) red_add_bf16x8(ylo_p + te.x, lo4.x, lo4.y, lo4.z, lo4.w);
          if (tok_hi >= 0) red_add_bf16x8(yhi_p + te.x, hi4.x, hi4.y, hi4.z, hi4.w);
        }
      }
    };
    int e = 0;
#pragma unroll 1
    for (; e < tiles_exp; ++e) {
      mbar_wait_bounded(full_bar(c_stage), c_parity, abort_flag);
      if (pass == 0 && e < 10) { B200_TRACE_POINT(12 + 2 * e) }
      expand_fn(e, stage_addr);
      if (pass == 0 && e < 10) { B200_TRACE_POINT(13 + 2 * e) }
      __syncwarp();
      if (lane == 0) mbar_arrive_relaxed(empty_bar(c_stage));
      advance();
    }
    if (pass == 0) { B200_TRACE_POINT(10) }
  }
  B200_TRACE_POINT(11)
  if (tid == 0 && *abort_flag != 0) atomicOr(&g_b200_status, kStatusWaitGaveUp);
}

// ------------------------------------------------------------------ host side
struct BgmvOptions {
  int cluster = 0;   // 0 = auto
  int pdl = 1;
  int ring_kb = 0;   // cap of the stage ring in KB (0 = default)
  int ksplit = 1;    // 1 = deal K parts over the cluster when the input rows are long enough (default)
};
inline BgmvOptions& bgmv_options() {
  static BgmvOptions o;
  return o;
}
// Default budget of one CTA: half of an SM's shared memory (228 KB minus 1 KB that the system keeps per
// resident CTA), so that a CTA of the next launch fits beside one of this launch.
constexpr int kBgmvSmemCoResident = (228 * 1024 - 2 * 1024) / 2;

inline bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }
inline int floor_pow2(int v) { int r = 1; while (r * 2 <= v) r *= 2; return r; }
inline int log2_exact(int v) { int s = 0; while ((1 << s) < v) ++s; return s; }

// Fills `pp` with the tiling for this problem; returns false (and a reason) when
// the fused kernel cannot run it.
inline bool bgmv_plan(const BgmvProblem& b, BgmvParams* pp, const char** why) {
  const char* dummy;
  if (why == nullptr) why = &dummy;
  SliceTable st;
  st.n = 0;
  for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) { st.a[s] = st.b[s] = nullptr; st.out[s] = st.col[s] = 0; }
  for (int s = 0; s < b.st.n; ++s) {
    if (b.st.out[s] == 0) continue;
    st.a[st.n] = b.st.a[s]; st.b[st.n] = b.st.b[s]; st.out[st.n] = b.st.out[s]; st.col[st.n] = b.st.col[s];
    ++st.n;
  }
  if (st.n == 0) { *why = "no active slice"; return false; }
  if (b.r_max % 32 != 0 || b.r_max > 256) { *why = "r_max must be a multiple of 32, <= 256"; return false; }
  if (b.in_dim % 32 != 0) { *why = "in_dim must be a multiple of 32"; return false; }
  if (b.x_ld % 8 != 0 || b.y_ld % 8 != 0) { *why = "row strides must be multiples of 8 elements"; return false; }
  if (!aligned16(b.x) || !aligned16(b.y)) { *why = "x / y must be 16-byte aligned"; return false; }
  for (int s = 0; s < st.n; ++s) {
    if (st.out[s] % 8 != 0 || st.col[s] % 8 != 0) { *why = "slice widths / offsets must be multiples of 8"; return false; }
    if (!aligned16(st.a[s]) || !aligned16(st.b[s])) { *why = "slabs must be 16-byte aligned"; return false; }
  }
  if (b.n_buckets < 1 || b.n_buckets > 65535) { *why = "n_buckets outside [1, 65535]"; return false; }

  const int Q = st.n * b.r_max;
  int C = bgmv_options().cluster;
  if (C != 1 && C != 2 && C != 4 && C != 8) {
    // Buckets expected to hold rows: graph buffers carry one bucket per slot, most of them empty, and a bucket
    // without rows exits at once. With T rows dealt over nb buckets about nb * (1 - exp(-T / nb)) are in use.
    // 4 CTAs per bucket while two consecutive launches fit side by side (296 CTAs are resident at two per SM), then
    // 2, then 1. Measured on a 24-layer decoder step of 64 rows over 129 buckets (about 30 in use): 2.13 ms per step
    // with clusters of 4, 2.27 with 2, 2.42 with 1, 2.46 with 8; on 256 rows over 33 buckets 4.9 us per launch with
    // 4, 7.0 with 2, 6.8 with 8.
    const double nb = (double)b.n_buckets;
    const double in_use = nb * (1.0 - std::exp(-(double)std::max(b.T, 1) / nb));
    C = in_use <= 56.0 ? 4 : (in_use <= 112.0 ? 2 : 1);
    // Large adapters (rank 64 on 4096-wide layers: 1 - 5 MB per bucket) keep an SM busy for tens of microseconds;
    // then the balance over the SMs matters more than room for the next launch: at most 512 KB of slab per CTA.
    // Measured on a 4-layer slice of a 32-head decoder, 512 rows over 175 adapters: 20.8 ms per step with one CTA
    // per bucket, 19.7 with 2, 19.0 with 4.
    int64_t bucket_bytes = 0;
    for (int s = 0; s < st.n; ++s) bucket_bytes += 2 * (int64_t)b.r_max * ((int64_t)b.in_dim + st.out[s]);
    while (C < 4 && bucket_bytes / C > 512 * 1024) C *= 2;
  }
  // K split: at least one K part (1024 columns) per CTA of the cluster and all rank rows in one CTA;
  // the shrink-only / expand-only pair of the tensor-parallel exchange keeps the row split
  const int nkp_all = ceil_div_i(b.in_dim, kBgmvKP);
  const bool ksplit = bgmv_options().ksplit && C > 1 && (b.mode == 0 || b.mode == 3) && nkp_all >= C && Q <= kBgmvMaxRc;
  if (!ksplit)
    while (C < 8 && round_up_i(ceil_div_i(Q, C), 8) > kBgmvMaxRc) C *= 2;
  const int Rc = ksplit ? Q : round_up_i(ceil_div_i(Q, C), 8);
  if (Rc > kBgmvMaxRc) { *why = "n_slices * r_max too large for one cluster"; return false; }

  BgmvParams p;
  p.y = static_cast<__nv_bfloat16*>(b.y); p.y_ld = b.y_ld;
  p.x = static_cast<const __nv_bfloat16*>(b.x); p.x_ld = b.x_ld;
  p.T = b.T; p.in_dim = b.in_dim; p.S = b.S; p.r_max = b.r_max; p.st = st;
  p.rank_per_slot = b.rank_per_slot; p.scale_per_slot = b.scale_per_slot;
  p.sorted_idx = b.sorted_idx; p.slot_ids = b.slot_ids; p.counts = b.counts; p.offsets = b.offsets;
  p.n_buckets = b.n_buckets; p.scaling = b.scaling;
  p.c_shift = log2_exact(C);
  p.KP = std::min(b.in_dim, kBgmvKP);
  p.nkp = ceil_div_i(b.in_dim, p.KP);
  p.pitchA = p.KP * 2 + (p.nkp > 1 ? 64 : 0);  // dense when a tile is one contiguous copy
  const int stageA = 8 * p.pitchA;
  p.ER = std::max(32, std::min(256, floor_pow2(16384 / (b.r_max * 2))));
  p.er_shift = log2_exact(p.ER);
  int tiles = (Rc / 8) * (ksplit ? ceil_div_i(p.nkp, C) : p.nkp);
  for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) p.oc[s] = 0;
  for (int s = 0; s < st.n; ++s) {
    p.oc[s] = round_up_i(ceil_div_i(st.out[s], C), 32);
    tiles += ceil_div_i(p.oc[s], p.ER);
  }
  const int stageB = p.ER * b.r_max * 2;
  p.stage_bytes = round_up_i(std::max(stageA, stageB), 128);
  // floats per token row: a multiple of 4 (16-byte reads) that is 8 modulo 16, so that the eight token
  // rows of a half warp start in different banks
  p.red_pitch = (Rc % 16 == 8) ? Rc : Rc + 8;
  const int red_bytes = round_up_i(kBgmvWarps * kBgmvTok * p.red_pitch * 4, 128);
  p.pitchT = round_up_i(Q * 2, 128) + 64;
  p.tmp_bytes = round_up_i(kBgmvTok * p.pitchT, 128);
  const int bar_bytes = 256;
  int exp_tiles = 0;
  for (int s = 0; s < st.n; ++s) exp_tiles += ceil_div_i(p.oc[s], p.ER);
  if (exp_tiles > kBgmvMaxExpandTiles) { *why = "too many expand tiles per CTA"; return false; }
  const int tab_bytes = round_up_i(std::max(exp_tiles, 1) * 8, 128);
  p.ksplit = ksplit ? 1 : 0;
  p.pitchR = Q + 4;
  p.recv_bytes = ksplit ? C * kBgmvTok * p.pitchR * 4 : 0;
  const int fixed = red_bytes + 2 * p.tmp_bytes + 2 * p.recv_bytes + tab_bytes + bar_bytes;
  // ring: what fits beside a second CTA on the SM, unless the caller set a size (up to the whole SM)
  const int ring_bytes = bgmv_options().ring_kb > 0 ? bgmv_options().ring_kb * 1024
                                                    : std::max(kBgmvSmemCoResident - fixed - 256, 2 * p.stage_bytes);
  int NS = std::min(std::max(tiles, 2), (kBgmvSmemMax - fixed - 256) / p.stage_bytes);
  NS = std::min(NS, kBgmvMaxStages);
  NS = std::min(NS, std::max(2, ring_bytes / p.stage_bytes));
  if (NS < 2) { *why = "shared memory too small for two stages"; return false; }
  p.NS = NS;
  p.off_red = NS * p.stage_bytes;
  p.off_tmp = p.off_red + red_bytes;
  p.off_recv = p.off_tmp + 2 * p.tmp_bytes;
  p.off_tab = p.off_recv + 2 * p.recv_bytes;
  p.off_bar = p.off_tab + tab_bytes;
  p.full_k = (p.KP == kBgmvKP && b.in_dim % kBgmvKP == 0) ? 1 : 0;
  p.y_cols = 0;
  for (int s = 0; s < st.n; ++s) p.y_cols = std::max(p.y_cols, st.col[s] + st.out[s]);
  p.use_pdl = bgmv_options().pdl ? 1 : 0;
  p.mode = b.mode;
  p.tmp_io = b.tmp_io;
  p.token_to_slot = b.token_to_slot;
  if ((b.mode == 1 || b.mode == 2) && b.tmp_io == nullptr) { *why = "shrink-only / expand-only need the tmp array"; return false; }
  if (b.mode == 3 && b.token_to_slot == nullptr) { *why = "overwrite mode needs token_to_slot"; return false; }
  if (pp != nullptr) *pp = p;
  return true;
}

inline bool bgmv_supported(const BgmvProblem& b, const char** why) { return bgmv_plan(b, nullptr, why); }

inline int bgmv_launch(const BgmvProblem& b, cudaStream_t stream) {
  BgmvParams p;
  const char* why = nullptr;
  if (!bgmv_plan(b, &p, &why)) return fail(B200_LORA_EUNSUPPORTED, "fused decode kernel: %s", why);
  const size_t smem = (size_t)p.off_bar + 256;
  static thread_local int configured_device = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_device != dev) {
    const void* kernels[8] = {(const void*)bgmv_fused_kernel<0, false>, (const void*)bgmv_fused_kernel<0, true>,
                              (const void*)bgmv_fused_kernel<1, false>, (const void*)bgmv_fused_kernel<1, true>,
                              (const void*)bgmv_fused_kernel<2, false>, (const void*)bgmv_fused_kernel<2, true>,
                              (const void*)bgmv_fused_kernel<3, false>, (const void*)bgmv_fused_kernel<3, true>};
    for (const void* k : kernels) {
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kBgmvSmemMax);
      if (e != cudaSuccess) return fail(B200_LORA_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    configured_device = dev;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1u << p.c_shift, (unsigned)p.n_buckets, 1);
  cfg.blockDim = dim3(kBgmvThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  attrs[na].id = cudaLaunchAttributeClusterDimension;
  attrs[na].val.clusterDim.x = 1u << p.c_shift;
  attrs[na].val.clusterDim.y = 1;
  attrs[na].val.clusterDim.z = 1;
  ++na;
  if (p.use_pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = (unsigned)na;
  cudaError_t e;
#define B200_BGMV_LAUNCH(M) \
  (p.full_k ? cudaLaunchKernelEx(&cfg, bgmv_fused_kernel<M, true>, p) : cudaLaunchKernelEx(&cfg, bgmv_fused_kernel<M, false>, p))
  switch (p.mode) {
    case 1: e = B200_BGMV_LAUNCH(1); break;
    case 2: e = B200_BGMV_LAUNCH(2); break;
    case 3: e = B200_BGMV_LAUNCH(3); break;
    default: e = B200_BGMV_LAUNCH(0); break;
  }
#undef B200_BGMV_LAUNCH
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(B200_LORA_ECUDA, "bgmv_fused_kernel launch: %s", cudaGetErrorString(e));
  }
  return B200_LORA_OK;
}

}  // namespace b200lora
