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
//   distributed shared memory between the two phases.
//
// Data movement
//   All weight and activation rows reach shared memory through 1-D bulk async copies
//   (cp.async.bulk, the TMA unit) into a ring of stages guarded by full/empty
//   mbarriers; warp 0 issues the copies NS-1 tiles ahead, so at kernel start the
//   CTA's first NS tiles (usually all of its weights) are in flight at once. The
//   weights do not depend on the previous kernel in the stream, so with programmatic
//   dependent launch their copies are issued before griddepcontrol.wait.
//
// Math
//   mma.sync m16n8k16 bf16 -> fp32 with tokens as the 16-row operand (a pass handles
//   16 tokens of the bucket) and weight rows as the 8-column operand. Fragments are
//   read as 16-byte vectors: thread (g,t) of a warp takes columns [8t, 8t+8) of a
//   32-column block for both operands, which is a fixed permutation of the k index
//   shared by A and B and therefore leaves the dot products unchanged.
//
// Rows whose slot is -1 are in no bucket and are never read or written.
#pragma once

#include "common.cuh"
#include "ptx.cuh"

namespace b200lora {

constexpr int kBgmvWarps = 8;
constexpr int kBgmvThreads = kBgmvWarps * 32;
constexpr int kBgmvTok = 16;            // tokens per pass (one MMA M tile)
constexpr int kBgmvMaxRc = 48;          // stacked rank rows per CTA
constexpr int kBgmvStageMax = 40 * 1024;
constexpr int kBgmvSmemMax = 232448;    // 227 KB opt-in maximum per CTA

// status bits of the device status word
constexpr int kStatusWaitGaveUp = 1;

__device__ int g_b200_status = 0;

struct BgmvProblem {
  void* y; int64_t y_ld; const void* x; int64_t x_ld;
  int T, in_dim, S, r_max;
  SliceTable st;
  const int32_t* rank_per_slot; const float* scale_per_slot;
  const int32_t *sorted_idx, *slot_ids, *counts, *offsets;
  int n_buckets; float scaling;
};

struct BgmvParams {
  __nv_bfloat16* y; int64_t y_ld; const __nv_bfloat16* x; int64_t x_ld;
  int T, in_dim, S, r_max;
  SliceTable st;  // active slices only
  const int32_t* rank_per_slot; const float* scale_per_slot;
  const int32_t *sorted_idx, *slot_ids, *counts, *offsets;
  int n_buckets; float scaling;
  int C;            // cluster size
  int KC;           // shrink K chunk per tile (256 or 512)
  int pitchA;       // bytes between rows of a shrink tile (KC*2 + 64)
  int ER;           // out rows per expand tile (multiple of 32)
  int stage_bytes, NS;
  int red_pitch;    // floats per token row of the cross-warp reduction buffer
  int pitchT;       // bytes per token row of tmp
  int off_red, off_tmp, off_bar;
  int use_pdl;
};

__host__ __device__ __forceinline__ int ceil_div_i(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ __forceinline__ int round_up_i(int a, int b) { return ceil_div_i(a, b) * b; }

__global__ void __launch_bounds__(kBgmvThreads, 1) bgmv_fused_kernel(const __grid_constant__ BgmvParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int bucket = blockIdx.y;
  const int C = p.C;
  const int c = (int)cluster_ctarank();

  // ---- bucket metadata (uniform across the cluster) -------------------------
  const int slot = p.slot_ids[bucket];
  const int cnt = p.counts[bucket];
  const int start = p.offsets[bucket];
  if (slot < 0 || slot >= p.S || cnt <= 0 || start < 0 || start > p.T - cnt) return;
  int rank = p.r_max;
  if (p.rank_per_slot != nullptr) rank = min(max(p.rank_per_slot[slot], 0), p.r_max);
  const int r_eff = min(p.r_max, (rank + 31) & ~31);
  if (r_eff == 0) return;
  const float sc = p.scaling * (p.scale_per_slot != nullptr ? p.scale_per_slot[slot] : 1.0f);

  const int n = p.st.n;
  const int in_dim = p.in_dim;
  const int Q = n * r_eff;                                  // stacked rank rows
  const int Rc = round_up_i(ceil_div_i(Q, C), 8);           // rows owned per CTA
  const int q_lo = min(c * Rc, Q);
  const int rows_c = min(q_lo + Rc, Q) - q_lo;              // multiple of 8, may be 0
  const int nt_c = rows_c >> 3;                             // 8-row MMA column tiles
  const int KC = p.KC, pitchA = p.pitchA, ER = p.ER;
  const int nkt_c = rows_c > 0 ? ceil_div_i(in_dim, KC) : 0;
  int e_lo[B200_LORA_MAX_SLICES], e_n[B200_LORA_MAX_SLICES], e_tiles[B200_LORA_MAX_SLICES];
  int tiles_exp = 0;
#pragma unroll
  for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) {
    e_lo[s] = e_n[s] = e_tiles[s] = 0;
    if (s < n) {
      const int out = p.st.out[s];
      const int Oc = round_up_i(ceil_div_i(out, C), 32);
      e_lo[s] = min(c * Oc, out);
      e_n[s] = min(e_lo[s] + Oc, out) - e_lo[s];
      e_tiles[s] = ceil_div_i(e_n[s], ER);
      tiles_exp += e_tiles[s];
    }
  }
  const int tpp = nkt_c + tiles_exp;  // tiles per pass
  const int npass = ceil_div_i(cnt, kBgmvTok);
  const int total = tpp * npass;
  const int NS = p.NS;

  uint8_t* ring = smem;
  float* red = reinterpret_cast<float*>(smem + p.off_red);
  uint8_t* tmp_full = smem + p.off_tmp;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.off_bar);  // full[NS], empty[NS]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * NS);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (uint32_t)(NS + s); };

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), kBgmvWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  cluster_arrive();  // peers are running once this completes (waited before the first remote store)

  // ---- tile issue (warp 0) -----------------------------------------------------
  // part bit 0: weight rows, bit 1: activation rows. A shrink tile's full barrier
  // takes expect_tx for the weights and arrive.expect_tx for the activations, so the
  // two halves may be issued at different times.
  auto issue_tile = [&](int it, int part) {
    const int stage = it % NS;
    const uint32_t sbase = smem_u32(ring + (size_t)stage * p.stage_bytes);
    const uint32_t fb = full_bar(stage);
    const int pass = it / tpp;
    int li = it - pass * tpp;
    if (li < nkt_c) {
      const int k0 = li * KC;
      const uint32_t row_bytes = (uint32_t)min(KC, in_dim - k0) * 2u;
      const int ntok = min(kBgmvTok, cnt - pass * kBgmvTok);
      if (part & 1) {
        if (lane == 0) mbar_expect_tx(fb, (uint32_t)rows_c * row_bytes);
        __syncwarp();
        for (int i = lane; i < rows_c; i += 32) {
          const int q = q_lo + i;
          const int s = q / r_eff, j = q - s * r_eff;
          const __nv_bfloat16* src =
              static_cast<const __nv_bfloat16*>(p.st.a[s]) + ((int64_t)slot * p.r_max + j) * in_dim + k0;
          bulk_g2s(sbase + (uint32_t)(i * pitchA), src, row_bytes, fb);
        }
      }
      if (part & 2) {
        if (lane == 0) mbar_arrive_expect_tx(fb, (uint32_t)ntok * row_bytes);
        __syncwarp();
        for (int i = lane; i < ntok; i += 32) {
          int tok = p.sorted_idx[start + pass * kBgmvTok + i];
          tok = min(max(tok, 0), p.T - 1);
          bulk_g2s(sbase + (uint32_t)((rows_c + i) * pitchA), p.x + (int64_t)tok * p.x_ld + k0, row_bytes, fb);
        }
      }
    } else if (part & 1) {
      li -= nkt_c;
      int s_sel = 0;
#pragma unroll
      for (int s = 0; s < B200_LORA_MAX_SLICES - 1; ++s) {
        if (s_sel == s && li >= e_tiles[s]) { li -= e_tiles[s]; s_sel = s + 1; }
      }
      int lo = 0, en = 0, out = 0;
      const void* bptr = nullptr;
#pragma unroll
      for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) {
        if (s == s_sel) { lo = e_lo[s]; en = e_n[s]; out = p.st.out[s]; bptr = p.st.b[s]; }
      }
      const int r0 = li * ER;
      const int nrows = min(ER, en - r0);
      if (lane == 0) {
        const uint32_t bytes = (uint32_t)nrows * (uint32_t)p.r_max * 2u;
        mbar_arrive_expect_tx(fb, bytes);
        const __nv_bfloat16* src =
            static_cast<const __nv_bfloat16*>(bptr) + ((int64_t)slot * out + lo + r0) * p.r_max;
        bulk_g2s(sbase, src, bytes, fb);
      }
    }
    __syncwarp();
  };

  // ---- prologue: weights first (independent of the previous kernel) ----------------
  const int npro = min(NS, total);
  if (warp == 0) {
    for (int it = 0; it < npro; ++it) issue_tile(it, 1);
  }
  if (p.use_pdl) {
    griddep_wait();
    griddep_launch_dependents();
  }
  if (warp == 0) {
    for (int it = 0; it < npro; ++it) issue_tile(it, 2);
  }

  int it = 0;  // global tile counter, identical in every thread
  for (int pass = 0; pass < npass; ++pass) {
    const bool valid_lo = pass * kBgmvTok + g < cnt;
    const bool valid_hi = pass * kBgmvTok + g + 8 < cnt;

    // ===== shrink: acc[j] = x[16 tok, K slice of this warp] . A_rows[8j..8j+8)^T =====
    float acc[kBgmvMaxRc / 8][4];
#pragma unroll
    for (int j = 0; j < kBgmvMaxRc / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    for (int kt = 0; kt < nkt_c; ++kt, ++it) {
      const int stage = it % NS;
      // refill the stage freed by the previous tile
      if (warp == 0 && it >= 1 && it - 1 + NS < total) {
        const int prev = it - 1;
        mbar_wait_bounded(empty_bar(prev % NS), (uint32_t)((prev / NS) & 1), abort_flag);
        issue_tile(prev + NS, 3);
      }
      mbar_wait_bounded(full_bar(stage), (uint32_t)((it / NS) & 1), abort_flag);
      const uint32_t sbase = smem_u32(ring + (size_t)stage * p.stage_bytes);
      const int k0 = kt * KC;
      const int nblk = min(KC, in_dim - k0) >> 5;  // 32-column blocks in this tile
      for (int b = warp; b < nblk; b += kBgmvWarps) {
        const uint32_t coff = (uint32_t)(b * 32 + t * 8) * 2u;
        uint4 xlo = make_uint4(0, 0, 0, 0), xhi = make_uint4(0, 0, 0, 0);
        if (valid_lo) xlo = lds128(sbase + (uint32_t)((rows_c + g) * pitchA) + coff);
        if (valid_hi) xhi = lds128(sbase + (uint32_t)((rows_c + g + 8) * pitchA) + coff);
#pragma unroll
        for (int j = 0; j < kBgmvMaxRc / 8; ++j) {
          if (j < nt_c) {
            const uint4 w = lds128(sbase + (uint32_t)((8 * j + g) * pitchA) + coff);
            mma_bf16_16816(acc[j], xlo.x, xhi.x, xlo.y, xhi.y, w.x, w.y);
            mma_bf16_16816(acc[j], xlo.z, xhi.z, xlo.w, xhi.w, w.z, w.w);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(stage));
    }

    // ===== cross-warp reduction of the K slices, scale, bf16, all-gather =====
    if (rows_c > 0) {
#pragma unroll
      for (int j = 0; j < kBgmvMaxRc / 8; ++j) {
        if (j < nt_c) {
          float* r0 = red + ((size_t)warp * kBgmvTok + g) * p.red_pitch + 8 * j + 2 * t;
          float* r1 = red + ((size_t)warp * kBgmvTok + g + 8) * p.red_pitch + 8 * j + 2 * t;
          *reinterpret_cast<float2*>(r0) = make_float2(acc[j][0], acc[j][1]);
          *reinterpret_cast<float2*>(r1) = make_float2(acc[j][2], acc[j][3]);
        }
      }
    }
    __syncthreads();
    cluster_wait();  // pairs with the arrive at kernel start / end of the previous pass
    {
      const int half = rows_c >> 1;
      for (int idx = tid; idx < kBgmvTok * half; idx += kBgmvThreads) {
        const int tok = idx / half, pr = idx - tok * half;
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int w = 0; w < kBgmvWarps; ++w) {
          const float2 v = *reinterpret_cast<const float2*>(red + ((size_t)w * kBgmvTok + tok) * p.red_pitch + 2 * pr);
          s0 += v.x;
          s1 += v.y;
        }
        const uint32_t v = pack_bf16x2(s0 * sc, s1 * sc);
        const uint32_t laddr = smem_u32(tmp_full + (size_t)tok * p.pitchT + (size_t)(q_lo + 2 * pr) * 2);
        for (int rc = 0; rc < C; ++rc) st_cluster_u32(mapa_shared(laddr, (uint32_t)rc), v);
      }
    }
    cluster_arrive();
    cluster_wait();

    // ===== expand: y[tok, cols] += tmp[16 tok, r] . B_rows^T ======================
    int tok_lo = -1, tok_hi = -1;
    if (valid_lo) tok_lo = p.sorted_idx[start + pass * kBgmvTok + g];
    if (valid_hi) tok_hi = p.sorted_idx[start + pass * kBgmvTok + g + 8];
    if (tok_lo >= p.T) tok_lo = -1;
    if (tok_hi >= p.T) tok_hi = -1;
    const uint32_t tmp_lo = smem_u32(tmp_full + (size_t)g * p.pitchT);
    const uint32_t tmp_hi = smem_u32(tmp_full + (size_t)(g + 8) * p.pitchT);
    const uint32_t pitchB = (uint32_t)p.r_max * 2u;
    const int kblocks = r_eff >> 5;

#pragma unroll
    for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) {
      if (s >= n) continue;
      for (int et = 0; et < e_tiles[s]; ++et, ++it) {
        const int stage = it % NS;
        if (warp == 0 && it >= 1 && it - 1 + NS < total) {
          const int prev = it - 1;
          mbar_wait_bounded(empty_bar(prev % NS), (uint32_t)((prev / NS) & 1), abort_flag);
          issue_tile(prev + NS, 3);
        }
        mbar_wait_bounded(full_bar(stage), (uint32_t)((it / NS) & 1), abort_flag);
        const uint32_t sbase = smem_u32(ring + (size_t)stage * p.stage_bytes);
        const int r0 = et * ER;
        const int nrows = min(ER, e_n[s] - r0);
        const int nblocks = ceil_div_i(nrows, 32);
        const int col0 = p.st.col[s] + e_lo[s] + r0;
        for (int blk = warp; blk < nblocks; blk += kBgmvWarps) {
          float d[4][4];
#pragma unroll
          for (int j = 0; j < 4; ++j) d[j][0] = d[j][1] = d[j][2] = d[j][3] = 0.f;
          const int rb = blk * 32;
          for (int kb = 0; kb < kblocks; ++kb) {
            const uint32_t koff = (uint32_t)(s * r_eff + kb * 32 + t * 8) * 2u;
            const uint4 alo = lds128(tmp_lo + koff);
            const uint4 ahi = lds128(tmp_hi + koff);
            const uint32_t woff = (uint32_t)(kb * 32 + t * 8) * 2u;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              // MMA column n of tile j reads slab row 8*(n/2) + 2j + (n%2): thread (g,t)
              // then owns 8 consecutive output columns 8t..8t+7 of the block.
              const int prow = rb + 8 * (g >> 1) + 2 * j + (g & 1);
              const uint4 w = lds128(sbase + (uint32_t)prow * pitchB + woff);
              mma_bf16_16816(d[j], alo.x, ahi.x, alo.y, ahi.y, w.x, w.y);
              mma_bf16_16816(d[j], alo.z, ahi.z, alo.w, ahi.w, w.z, w.w);
            }
          }
          if (rb + 8 * t < nrows) {
            const int col = col0 + rb + 8 * t;
            if (tok_lo >= 0) {
              uint4* yp = reinterpret_cast<uint4*>(p.y + (int64_t)tok_lo * p.y_ld + col);
              uint4 v = *yp;
              v.x = pack_bf16x2(bf16_lo(v.x) + d[0][0], bf16_hi(v.x) + d[0][1]);
              v.y = pack_bf16x2(bf16_lo(v.y) + d[1][0], bf16_hi(v.y) + d[1][1]);
              v.z = pack_bf16x2(bf16_lo(v.z) + d[2][0], bf16_hi(v.z) + d[2][1]);
              v.w = pack_bf16x2(bf16_lo(v.w) + d[3][0], bf16_hi(v.w) + d[3][1]);
              *yp = v;
            }
            if (tok_hi >= 0) {
              uint4* yp = reinterpret_cast<uint4*>(p.y + (int64_t)tok_hi * p.y_ld + col);
              uint4 v = *yp;
              v.x = pack_bf16x2(bf16_lo(v.x) + d[0][2], bf16_hi(v.x) + d[0][3]);
              v.y = pack_bf16x2(bf16_lo(v.y) + d[1][2], bf16_hi(v.y) + d[1][3]);
              v.z = pack_bf16x2(bf16_lo(v.z) + d[2][2], bf16_hi(v.z) + d[2][3]);
              v.w = pack_bf16x2(bf16_lo(v.w) + d[3][2], bf16_hi(v.w) + d[3][3]);
              *yp = v;
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(stage));
      }
    }
    // tmp of this pass is no longer needed: peers may overwrite it in the next pass
    if (pass + 1 < npass) cluster_arrive();
  }
  if (tid == 0 && *abort_flag != 0) atomicOr(&g_b200_status, kStatusWaitGaveUp);
}

// ------------------------------------------------------------------ host side
struct BgmvOptions {
  int cluster = 0;  // 0 = auto
  int pdl = 1;
};
inline BgmvOptions& bgmv_options() {
  static BgmvOptions o;
  return o;
}

inline bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

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
    C = b.n_buckets <= 37 ? 4 : (b.n_buckets <= 74 ? 2 : 1);
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
  p.C = C;
  const int rows_stage = Rc + kBgmvTok;
  p.KC = (b.in_dim >= 512 && rows_stage * (512 * 2 + 64) <= kBgmvStageMax) ? 512 : 256;
  p.pitchA = p.KC * 2 + 64;
  const int stageA = rows_stage * p.pitchA;
  int oc_max = 0, tiles = ceil_div_i(b.in_dim, p.KC);
  for (int s = 0; s < st.n; ++s) oc_max = std::max(oc_max, round_up_i(ceil_div_i(st.out[s], C), 32));
  p.ER = std::min(oc_max, (kBgmvStageMax / (b.r_max * 2)) / 32 * 32);
  for (int s = 0; s < st.n; ++s) tiles += ceil_div_i(round_up_i(ceil_div_i(st.out[s], C), 32), p.ER);
  const int stageB = p.ER * b.r_max * 2;
  p.stage_bytes = round_up_i(std::max(stageA, stageB), 1024);
  p.red_pitch = Rc + 2;
  const int red_bytes = round_up_i(kBgmvWarps * kBgmvTok * p.red_pitch * 4, 128);
  p.pitchT = round_up_i(Q * 2, 128) + 64;
  const int tmp_bytes = round_up_i(kBgmvTok * p.pitchT, 128);
  const int bar_bytes = 256;
  const int fixed = red_bytes + tmp_bytes + bar_bytes;
  int NS = std::min(std::max(tiles, 2), (kBgmvSmemMax - fixed) / p.stage_bytes);
  NS = std::min(NS, 12);
  if (NS < 2) { *why = "shared memory too small for two stages"; return false; }
  p.NS = NS;
  p.off_red = NS * p.stage_bytes;
  p.off_tmp = p.off_red + red_bytes;
  p.off_bar = p.off_tmp + tmp_bytes;
  p.use_pdl = bgmv_options().pdl ? 1 : 0;
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
    cudaError_t e = cudaFuncSetAttribute(bgmv_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBgmvSmemMax);
    if (e != cudaSuccess) return fail(B200_LORA_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured_device = dev;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)p.C, (unsigned)p.n_buckets, 1);
  cfg.blockDim = dim3(kBgmvThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  attrs[na].id = cudaLaunchAttributeClusterDimension;
  attrs[na].val.clusterDim.x = (unsigned)p.C;
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
  cudaError_t e = cudaLaunchKernelEx(&cfg, bgmv_fused_kernel, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(B200_LORA_ECUDA, "bgmv_fused_kernel launch: %s", cudaGetErrorString(e));
  }
  return B200_LORA_OK;
}

}  // namespace b200lora
