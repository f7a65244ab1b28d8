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

// status bits of the device status word
constexpr int kStatusWaitGaveUp = 1;

__device__ int g_b200_status = 0;

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
  int off_red, off_tmp, off_bar;
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

#ifndef BGMV_MINBLOCKS
#define BGMV_MINBLOCKS 1
#endif
#ifndef BGMV_YDEPTH
#define BGMV_YDEPTH 2
#endif
// kOverwrite = mode 3, compiled separately so that the add path carries none of its branches
template <bool kOverwrite>
__global__ void __launch_bounds__(kBgmvThreads, BGMV_MINBLOCKS) bgmv_fused_kernel(const __grid_constant__ BgmvParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int bucket = blockIdx.y;
  const int C = 1 << p.c_shift;
  const int c = (int)cluster_ctarank();
  const int NS = p.NS;

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
      mbar_init(tmp_ready_bars, (uint32_t)C);
      mbar_init(tmp_ready_bars + 8u, (uint32_t)C);
      *abort_flag = 0;
    }
    mbar_fence_init();
  }

  int rank = p.r_max;
  if (p.rank_per_slot != nullptr && slot >= 0 && slot < p.S) rank = min(max(p.rank_per_slot[slot], 0), p.r_max);
  const int r_eff = min(p.r_max, (rank + 31) & ~31);
  if (slot < 0 || slot >= p.S || cnt <= 0 || start < 0 || start > p.T - cnt || r_eff == 0) {
    if (kOverwrite) {  // an idle cluster still does its share of the -0.0 rows
      if (p.use_pdl) griddep_wait();
      bgmv_fill_rows_without_delta(p, bucket * C + c, (int)gridDim.y * C, tid, kBgmvThreads);
    }
    return;
  }
  const float sc = p.scaling * (p.scale_per_slot != nullptr ? p.scale_per_slot[slot] : 1.0f);
  B200_TRACE_POINT(1)

  const int n = p.st.n;
  const int in_dim = p.in_dim;
  const int Q = n * r_eff;                                       // stacked rank rows
  const int Rc = ((((Q + C - 1) >> p.c_shift) + 7) & ~7);        // rows owned per CTA
  const int q_lo = min(c * Rc, Q);
  const int mode = p.mode;
  const int rows_c = mode == 2 ? 0 : min(q_lo + Rc, Q) - q_lo;   // multiple of 8, may be 0 (expand only: no shrink rows)
  const int nt_c = rows_c >> 3;                                  // 8-row tiles of this CTA
  const int KP = p.KP, pitchA = p.pitchA, ER = p.ER, nkp = p.nkp;
  const int shrink_tiles = nt_c * nkp;
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
    for (int it = 0; it < total; ++it) {
      if (p_round > 0) mbar_wait_bounded(empty_bar(p_stage), (uint32_t)((p_round & 1) ^ 1), abort_flag);
      const uint32_t sbase = ring_base + (uint32_t)p_stage * (uint32_t)p.stage_bytes;
      const uint32_t fb = full_bar(p_stage);
      if (i_shrink) {
        const int k0 = i_kp * KP;
        const uint32_t row_bytes = (uint32_t)min(KP, in_dim - k0) * 2u;
        const void* aptr = nullptr;
#pragma unroll
        for (int s = 0; s < B200_LORA_MAX_SLICES; ++s)
          if (s == i_qs) aptr = p.st.a[s];
        const __nv_bfloat16* src =
            static_cast<const __nv_bfloat16*>(aptr) + ((int64_t)slot * p.r_max + i_qr) * in_dim + k0;
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
          if (++i_kp == nkp) { i_kp = 0; i_shrink = tiles_exp > 0 ? 0 : 1; i_s = 0; i_et = 0; }
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
      }
    }
    cluster_wait();
    return;
  }

  // ============================= consumer warps =============================
  // Token rows of the first pass (index metadata: safe before the wait). While the previous
  // kernel finishes, pull this CTA's activation rows and its first output columns into L2:
  // a prefetch never creates stale data (L2 is the point of coherence), it only hides the
  // HBM latency of rows nobody has touched recently.
  int tok0_lo = -1, tok0_hi = -1;
  if (g < cnt) tok0_lo = p.sorted_idx[start + g];
  if (g + 8 < cnt) tok0_hi = p.sorted_idx[start + g + 8];
  if (tok0_lo >= p.T) tok0_lo = -1;
  if (tok0_hi >= p.T) tok0_hi = -1;
  if (p.use_pdl) {
    if (rows_c > 0) {
      for (int kc = warp * 32 + t * 8; kc < in_dim; kc += kBgmvWarps * 32) {
        if (tok0_lo >= 0) prefetch_l2(p.x + (int64_t)tok0_lo * p.x_ld + kc);
        if (tok0_hi >= 0) prefetch_l2(p.x + (int64_t)tok0_hi * p.x_ld + kc);
      }
    }
#pragma unroll
    for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) {
      if (s < n && !kOverwrite) {
        for (int r = warp * 32 + t * 8; r < e_n[s]; r += kBgmvWarps * 32) {
          const int cc = p.st.col[s] + e_lo[s] + r;
          if (tok0_lo >= 0) prefetch_l2(p.y + (int64_t)tok0_lo * p.y_ld + cc);
          if (tok0_hi >= 0) prefetch_l2(p.y + (int64_t)tok0_hi * p.y_ld + cc);
        }
      }
    }
    griddep_wait();  // x and y of this launch are final from here on
  }
  if (kOverwrite) bgmv_fill_rows_without_delta(p, bucket * C + c, (int)gridDim.y * C, tid, kBgmvConsumers);
  B200_TRACE_POINT(4)

  int c_stage = 0, c_round = 0;  // stage / round of the tile being consumed
  auto advance = [&]() {
    if (++c_stage == NS) { c_stage = 0; ++c_round; }
  };
  const uint32_t pitchB = (uint32_t)p.r_max * 2u;
  const int kblocks = r_eff >> 5;

  for (int pass = 0; pass < npass; ++pass) {
    const bool valid_lo = pass * kBgmvTok + g < cnt;
    const bool valid_hi = pass * kBgmvTok + g + 8 < cnt;
    int tok_lo = tok0_lo, tok_hi = tok0_hi;
    if (pass > 0) {
      tok_lo = tok_hi = -1;
      if (valid_lo) tok_lo = p.sorted_idx[start + pass * kBgmvTok + g];
      if (valid_hi) tok_hi = p.sorted_idx[start + pass * kBgmvTok + g + 8];
      if (tok_lo >= p.T) tok_lo = -1;
      if (tok_hi >= p.T) tok_hi = -1;
    }

    // y of this CTA's expand tiles is requested two tiles ahead (the first two right here, before
    // the shrink), so the read-modify-write of y never waits for an L2 round trip.
    int ys = 0, yet = 0, yleft = tiles_exp;  // cursor of the next tile whose y gets requested
    auto y_next = [&](uint4& lo4, uint4& hi4, int& col_, int& nrows_, int& s_) {
      lo4 = hi4 = make_uint4(0, 0, 0, 0);
      col_ = 0; nrows_ = 0; s_ = 0;
      if (yleft <= 0) return;
      --yleft;
#pragma unroll
      for (int s = 0; s < B200_LORA_MAX_SLICES - 1; ++s)  // skip slices this CTA has no tiles of
        if (ys == s && yet >= e_tiles[s]) { ys = s + 1; yet = 0; }
      int lo = 0, en = 0, cb = 0;
#pragma unroll
      for (int s = 0; s < B200_LORA_MAX_SLICES; ++s)
        if (s == ys) { lo = e_lo[s]; en = e_n[s]; cb = p.st.col[s]; }
      const int r0 = yet << p.er_shift;
      nrows_ = min(ER, en - r0);
      col_ = cb + lo + r0;
      s_ = ys;
      ++yet;
      if (!kOverwrite && warp * 32 + 8 * t < nrows_) {  // (overwrite: y is not read, the delta is added to zeros)
        const int cc = col_ + warp * 32 + 8 * t;
        if (tok_lo >= 0) lo4 = ldg128(p.y + (int64_t)tok_lo * p.y_ld + cc);
        if (tok_hi >= 0) hi4 = ldg128(p.y + (int64_t)tok_hi * p.y_ld + cc);
      }
    };
    uint4 q0lo, q0hi, q1lo, q1hi;
    int q0col, q0rows, q0s, q1col, q1rows, q1s;
    y_next(q0lo, q0hi, q0col, q0rows, q0s);
#if BGMV_YDEPTH == 2
    y_next(q1lo, q1hi, q1col, q1rows, q1s);
#else
    q1lo = q1hi = make_uint4(0, 0, 0, 0); q1col = q1rows = q1s = 0;
#endif

    // ===== shrink: red[warp][tok][row] = x[16 tok, K blocks of this warp] . A_rows^T =====
    for (int kp = 0; kp < (rows_c > 0 ? nkp : 0); ++kp) {
      const int k0 = kp * KP;
      // activation fragments of this warp's 32-column blocks, kept for all row tiles
      uint4 xlo[kBgmvXBlocks], xhi[kBgmvXBlocks];
#pragma unroll
      for (int i = 0; i < kBgmvXBlocks; ++i) {
        const int kl = (warp + kBgmvWarps * i) * 32;
        const int kcol = k0 + kl + t * 8;
        xlo[i] = xhi[i] = make_uint4(0, 0, 0, 0);
        if (kl < KP && kcol < in_dim) {
          if (tok_lo >= 0) xlo[i] = ldg128_nc(p.x + (int64_t)tok_lo * p.x_ld + kcol);
          if (tok_hi >= 0) xhi[i] = ldg128_nc(p.x + (int64_t)tok_hi * p.x_ld + kcol);
        }
      }
      for (int j = 0; j < nt_c; ++j) {
        mbar_wait_bounded(full_bar(c_stage), (uint32_t)(c_round & 1), abort_flag);
        if (kp == 0 && j == 0 && pass == 0) { B200_TRACE_POINT(5) }
        const uint32_t sbase = ring_base + (uint32_t)c_stage * (uint32_t)p.stage_bytes;
        // two independent accumulator chains halve the dependent-MMA latency
        float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
        uint4 w[kBgmvXBlocks];
#pragma unroll
        for (int i = 0; i < kBgmvXBlocks; ++i) {
          const int kl = (warp + kBgmvWarps * i) * 32;
          w[i] = make_uint4(0, 0, 0, 0);
          if (kl < KP && k0 + kl < in_dim) w[i] = lds128(sbase + (uint32_t)(g * pitchA) + (uint32_t)(kl + t * 8) * 2u);
        }
#pragma unroll
        for (int i = 0; i < kBgmvXBlocks; ++i) {
          mma_bf16_16816(acc, xlo[i].x, xhi[i].x, xlo[i].y, xhi[i].y, w[i].x, w[i].y);
          mma_bf16_16816(acc2, xlo[i].z, xhi[i].z, xlo[i].w, xhi[i].w, w[i].z, w[i].w);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] += acc2[i];
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(c_stage));
        advance();
        // acc holds (tok g | g+8, rank rows 8j+2t, 8j+2t+1): accumulate over K parts per warp
        float2* r0 = reinterpret_cast<float2*>(red + ((size_t)warp * kBgmvTok + g) * p.red_pitch + 8 * j + 2 * t);
        float2* r1 = reinterpret_cast<float2*>(red + ((size_t)warp * kBgmvTok + g + 8) * p.red_pitch + 8 * j + 2 * t);
        if (kp == 0) {
          *r0 = make_float2(acc[0], acc[1]);
          *r1 = make_float2(acc[2], acc[3]);
        } else {
          const float2 a = *r0, b = *r1;
          *r0 = make_float2(a.x + acc[0], a.y + acc[1]);
          *r1 = make_float2(b.x + acc[2], b.y + acc[3]);
        }
      }
    }
    if (pass == 0) { B200_TRACE_POINT(6) }

    // ===== cross-warp reduction of the K slices, scale, bf16, all-gather =====
    named_bar_sync(1, kBgmvConsumers);
    if (pass == 0) {
      B200_TRACE_POINT(7)
      cluster_wait();  // start-up barrier: peers run and their barriers are initialised
    }
    uint8_t* tmp_full = tmp_base + (size_t)(pass & 1) * p.tmp_bytes;
    const uint32_t tmp_ready_bar = tmp_ready_bars + 8u * (uint32_t)(pass & 1);
    if (mode == 2) {
      // expand only: tmp of this pass comes from global memory (fp32 [n, T, r_max], summed over the
      // tensor-parallel ranks) and is rounded to bf16 into this CTA's own buffer
      const int tok = tid >> 4;
      int trow = -1;
      if (pass * kBgmvTok + tok < cnt) trow = p.sorted_idx[start + pass * kBgmvTok + tok];
      if (trow >= p.T) trow = -1;
      for (int pr = tid & 15; pr < (Q >> 1); pr += 16) {
        const int q = 2 * pr, s = q / r_eff, rr = q - s * r_eff;
        float2 v = make_float2(0.f, 0.f);
        if (trow >= 0) v = *reinterpret_cast<const float2*>(p.tmp_io + ((int64_t)s * p.T + trow) * p.r_max + rr);
        *reinterpret_cast<uint32_t*>(tmp_full + (size_t)tok * p.pitchT + (size_t)q * 2) = pack_bf16x2(v.x, v.y);
      }
      named_bar_sync(1, kBgmvConsumers);
    } else {
      const int half = rows_c >> 1;
      const int tok = tid >> 4;
      int trow = -1;  // shrink only: token row of `tok`
      if (mode == 1) {
        if (pass * kBgmvTok + tok < cnt) trow = p.sorted_idx[start + pass * kBgmvTok + tok];
        if (trow >= p.T) trow = -1;
      }
      for (int pr = tid & 15; pr < half; pr += 16) {
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int w = 0; w < kBgmvWarps; ++w) {
          const float2 v = *reinterpret_cast<const float2*>(red + ((size_t)w * kBgmvTok + tok) * p.red_pitch + 2 * pr);
          s0 += v.x;
          s1 += v.y;
        }
        if (mode == 1) {
          // shrink only: fp32 result of this CTA's rank rows straight to global memory
          const int q = q_lo + 2 * pr, s = q / r_eff, rr = q - s * r_eff;
          if (trow >= 0)
            *reinterpret_cast<float2*>(p.tmp_io + ((int64_t)s * p.T + trow) * p.r_max + rr) = make_float2(s0 * sc, s1 * sc);
        } else {
          const uint32_t v = pack_bf16x2(s0 * sc, s1 * sc);
          const uint32_t laddr = smem_u32(tmp_full + (size_t)tok * p.pitchT + (size_t)(q_lo + 2 * pr) * 2);
          for (int rc = 0; rc < C; ++rc) st_cluster_u32(mapa_shared(laddr, (uint32_t)rc), v);
        }
      }
      if (mode == 1) {
        named_bar_sync(1, kBgmvConsumers);  // all warps have read the reduction buffer before the next pass refills it
        continue;
      }
      named_bar_sync(1, kBgmvConsumers);  // every store of this CTA is issued
      if (tid < C) mbar_arrive_remote_release(mapa_shared(tmp_ready_bar, (uint32_t)tid));
      if (pass == 0) { B200_TRACE_POINT(8) }

      // ===== expand: y[tok, cols] += tmp[16 tok, r] . B_rows^T ======================
      mbar_wait_bounded_acquire_cluster(tmp_ready_bar, (uint32_t)((pass >> 1) & 1), abort_flag);
      if (pass == 0) { B200_TRACE_POINT(9) }
    }
    const uint32_t tmp_lo = smem_u32(tmp_full + (size_t)g * p.pitchT);
    const uint32_t tmp_hi = smem_u32(tmp_full + (size_t)(g + 8) * p.pitchT);

    for (int e = 0; e < tiles_exp; ++e) {
      // y of tile e was requested two tiles ago; request tile e+2 now
      const uint4 ylo = q0lo, yhi = q0hi;
      const int col = q0col, nrows = q0rows, s_cur = q0s;
#if BGMV_YDEPTH == 2
      q0lo = q1lo; q0hi = q1hi; q0col = q1col; q0rows = q1rows; q0s = q1s;
      y_next(q1lo, q1hi, q1col, q1rows, q1s);
#else
      y_next(q0lo, q0hi, q0col, q0rows, q0s);
#endif
      mbar_wait_bounded(full_bar(c_stage), (uint32_t)(c_round & 1), abort_flag);
      if (pass == 0 && e < 5) { B200_TRACE_POINT(12 + 4 * e) }
      const uint32_t sbase = ring_base + (uint32_t)c_stage * (uint32_t)p.stage_bytes;
      const int rb = warp * 32;  // ER <= 256: one 32-row block per warp and tile
      if (rb < nrows) {
        float d[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) d[j][0] = d[j][1] = d[j][2] = d[j][3] = 0.f;
        for (int kb = 0; kb < kblocks; ++kb) {
          const uint32_t koff = (uint32_t)(s_cur * r_eff + kb * 32 + t * 8) * 2u;
          const uint4 alo = lds128(tmp_lo + koff);
          const uint4 ahi = lds128(tmp_hi + koff);
          const uint32_t woff = (uint32_t)(kb * 32 + t * 8) * 2u;
          uint4 w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            // MMA column n of tile j reads slab row 8*(n/2) + 2j + (n%2): thread (g,t)
            // then owns 8 consecutive output columns 8t..8t+7 of the block.
            const int prow = rb + 8 * (g >> 1) + 2 * j + (g & 1);
            w[j] = lds128(sbase + (uint32_t)prow * pitchB + woff);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) mma_bf16_16816(d[j], alo.x, ahi.x, alo.y, ahi.y, w[j].x, w[j].y);
#pragma unroll
          for (int j = 0; j < 4; ++j) mma_bf16_16816(d[j], alo.z, ahi.z, alo.w, ahi.w, w[j].z, w[j].w);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(c_stage));  // the stage is in registers now
        if (pass == 0 && e < 5) { B200_TRACE_POINT(13 + 4 * e) }
        if (rb + 8 * t < nrows) {
          const int cc = col + rb + 8 * t;
          if (tok_lo >= 0) {
            uint4 v = ylo;
            v.x = add_bf16x2(v.x, d[0][0], d[0][1]);
            v.y = add_bf16x2(v.y, d[1][0], d[1][1]);
            v.z = add_bf16x2(v.z, d[2][0], d[2][1]);
            v.w = add_bf16x2(v.w, d[3][0], d[3][1]);
            stg128(p.y + (int64_t)tok_lo * p.y_ld + cc, v);
          }
          if (tok_hi >= 0) {
            uint4 v = yhi;
            v.x = add_bf16x2(v.x, d[0][2], d[0][3]);
            v.y = add_bf16x2(v.y, d[1][2], d[1][3]);
            v.z = add_bf16x2(v.z, d[2][2], d[2][3]);
            v.w = add_bf16x2(v.w, d[3][2], d[3][3]);
            stg128(p.y + (int64_t)tok_hi * p.y_ld + cc, v);
          }
        }
      } else {
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(c_stage));
      }
      if (pass == 0 && e < 5) { B200_TRACE_POINT(14 + 4 * e) }
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
};
inline BgmvOptions& bgmv_options() {
  static BgmvOptions o;
  return o;
}
constexpr int kBgmvDefaultRingKb = 200;  // as many tiles in flight as fit (measured best on B200)

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
    // buckets that can hold tokens: graph buffers carry one bucket per slot, most of them empty
    const int busy = std::min(b.n_buckets, std::max(b.T, 1));
    C = busy <= 37 ? 4 : (busy <= 74 ? 2 : 1);
  }
  while (C < 8 && round_up_i(ceil_div_i(Q, C), 8) > kBgmvMaxRc) C *= 2;
  const int Rc = round_up_i(ceil_div_i(Q, C), 8);
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
  int tiles = (Rc / 8) * p.nkp;
  for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) p.oc[s] = 0;
  for (int s = 0; s < st.n; ++s) {
    p.oc[s] = round_up_i(ceil_div_i(st.out[s], C), 32);
    tiles += ceil_div_i(p.oc[s], p.ER);
  }
  const int stageB = p.ER * b.r_max * 2;
  p.stage_bytes = round_up_i(std::max(stageA, stageB), 128);
  p.red_pitch = Rc + 2;
  const int red_bytes = round_up_i(kBgmvWarps * kBgmvTok * p.red_pitch * 4, 128);
  p.pitchT = round_up_i(Q * 2, 128) + 64;
  p.tmp_bytes = round_up_i(kBgmvTok * p.pitchT, 128);
  const int bar_bytes = 256;
  const int fixed = red_bytes + 2 * p.tmp_bytes + bar_bytes;
  const int ring_kb = bgmv_options().ring_kb > 0 ? bgmv_options().ring_kb : kBgmvDefaultRingKb;
  int NS = std::min(std::max(tiles, 2), (kBgmvSmemMax - fixed) / p.stage_bytes);
  NS = std::min(NS, kBgmvMaxStages);
  NS = std::min(NS, std::max(2, ring_kb * 1024 / p.stage_bytes));
  if (NS < 2) { *why = "shared memory too small for two stages"; return false; }
  p.NS = NS;
  p.off_red = NS * p.stage_bytes;
  p.off_tmp = p.off_red + red_bytes;
  p.off_bar = p.off_tmp + 2 * p.tmp_bytes;
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
    cudaError_t e = cudaFuncSetAttribute(bgmv_fused_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBgmvSmemMax);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(bgmv_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBgmvSmemMax);
    if (e != cudaSuccess) return fail(B200_LORA_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
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
  cudaError_t e = p.mode == 3 ? cudaLaunchKernelEx(&cfg, bgmv_fused_kernel<true>, p)
                              : cudaLaunchKernelEx(&cfg, bgmv_fused_kernel<false>, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(B200_LORA_ECUDA, "bgmv_fused_kernel launch: %s", cudaGetErrorString(e));
  }
  return B200_LORA_OK;
}

}  // namespace b200lora
