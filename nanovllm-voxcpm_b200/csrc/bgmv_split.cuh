// Fused decode multi-LoRA kernel, column-split variant (bf16): shrink + expand in ONE launch,
// sized so that TWO CTAs fit on an SM (<= 112 KB of shared memory, 160 threads). With
// programmatic dependent launch the CTAs of the next launch of the stream then become resident
// while this launch still computes, and pull their adapter weights (which no kernel of the stream
// writes) into shared memory before their griddepcontrol.wait returns: HBM stays busy across launch
// boundaries, and what is left after the wait is a short chain of on-chip steps.
//
// Work decomposition
//   grid = (C, n_buckets), cluster = (C, 1, 1): one cluster per slot bucket, as in bgmv_fused_kernel.
//   shrink : the INPUT columns are split across the C CTAs (Kc = in / C columns each, all n*r rank
//            rows). A stage of the ring is one tiled-TMA box of 32 rank rows x 256 columns of lora_A
//            (16 KB); warp w owns rank rows [8w, 8w+8) of every box, so no warp shares an
//            accumulator with another and nothing is reduced inside the CTA. Boxes arrive column
//            chunk by column chunk; a warp keeps the chunk's activation fragments in registers
//            for all boxes of the chunk.
//   exchange: every warp sends its fp32 partial sums to all C CTAs with st.async, which stores into
//            the peer's shared memory and counts the bytes on the peer's mbarrier in one operation
//            (no barrier + release/acquire round trip); each CTA then adds the C partials, scales,
//            rounds to bf16 once and holds tmp[16 tokens, n*r].
//   expand : each slice's output rows are split across the C CTAs; a stage is one contiguous copy of
//            up to 16 KB of lora_B rows. y is fetched with 16-byte cp.async into a per-thread staging
//            area several tiles ahead (each thread reads back only what it fetched itself, so no
//            barrier is involved) and written with 16-byte stores.
//   Activations x[16 tokens, Kc] are staged once per pass in shared memory by cp.async (L2 only:
//   the lines were prefetched into L2 before the wait, never into L1).
//
// Roles: warp 4 = producer (one thread issues the TMA copies into the full/empty ring),
// warps 0-3 = consumers (mma.sync m16n8k16, tokens as the 16-row operand). Every wait is bounded.
// Rows whose slot is -1 are in no bucket and are never read or written.
#pragma once

#include "bgmv_fused.cuh"
#include "tc_common.cuh"

namespace b200lora {

constexpr int kSplitWarps = 4;
constexpr int kSplitConsumers = kSplitWarps * 32;
constexpr int kSplitThreads = kSplitConsumers + 32;
constexpr int kSplitBoxRows = 32;
constexpr int kSplitBoxCols = 256;
constexpr int kSplitMaxStages = 12;
constexpr int kSplitMaxGroups = 4;   // 32-row lora_A boxes per column chunk (n_slices * r_max / 32)
#ifndef BGMV_SPLIT_YDEPTH
#define BGMV_SPLIT_YDEPTH 4
#endif
constexpr int kSplitYDepth = BGMV_SPLIT_YDEPTH;                 // y tiles in flight per thread
constexpr int kSplitYSlotBytes = 2 * 2 * kSplitConsumers * 16;  // 2 row blocks x (lo, hi) x 16 B per thread
constexpr int kSplitDefaultSmemKb = 112;                        // two CTAs per SM

struct BgmvSplitParams {
  __nv_bfloat16* y; int64_t y_ld; const __nv_bfloat16* x; int64_t x_ld;
  int T, in_dim, S, r_max;
  SliceTable st;  // active slices only
  const int32_t* rank_per_slot; const float* scale_per_slot;
  const int32_t *sorted_idx, *slot_ids, *counts, *offsets;
  int n_buckets; float scaling;
  int c_shift;         // cluster size C = 1 << c_shift
  int Kc;              // input columns per CTA (multiple of 32)
  int BC, nchunk;      // columns per lora_A box (<= 256) and boxes per Kc
  int a_stage_bytes;   // bytes of one lora_A box
  int ER, er_shift;    // out rows per expand tile (power of two, 32..256)
  int oc[B200_LORA_MAX_SLICES];  // out rows of each slice owned by one CTA (multiple of 32)
  int stage_bytes, NS;
  int pitchX;          // bytes per token row of the staged activations
  int pitchT;          // bytes per token row of tmp
  int pitchP;          // floats per token row of the received partial sums
  int off_x, off_y, off_recv, off_tmp, off_bar;
  int use_pdl;
};

struct BgmvSplitMaps {
  CUtensorMap a[B200_LORA_MAX_SLICES];  // lora_A slab s as a 2-D matrix [S * r_max, in]
};

__device__ __forceinline__ void st_async_f32x2(uint32_t cluster_addr, float a, float b, uint32_t cluster_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];" ::"r"(cluster_addr),
               "f"(a), "f"(b), "r"(cluster_bar)
               : "memory");
}
// 16-byte asynchronous copy global -> shared that bypasses L1
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void sts128_zero(uint32_t addr) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(addr), "r"(0u) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v));
}
__device__ __forceinline__ float2 lds_f32x2(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}

__global__ void __launch_bounds__(kSplitThreads, 2)
bgmv_split_kernel(const __grid_constant__ BgmvSplitParams p, const __grid_constant__ BgmvSplitMaps maps) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int bucket = blockIdx.y;
  const int C = 1 << p.c_shift;
  const int c = (int)cluster_ctarank();
  const int NS = p.NS;

  B200_TRACE_POINT(0)
  // The next launch of the stream may start at once: before its own wait it reads only index
  // metadata and lora slabs.
  if (p.use_pdl) griddep_launch_dependents();
  const int slot = p.slot_ids[bucket];
  const int cnt = p.counts[bucket];
  const int start = p.offsets[bucket];

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.off_bar);  // full[], empty[], part_ready, recv_free
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * kSplitMaxStages + 2);
  int* tab = reinterpret_cast<int*>(smem + p.off_bar + 256);       // e_lo[4], e_n[4], e_tiles[4], first y column[4]
  const uint32_t bar_base = smem_u32(bars);
  const uint32_t ring_base = smem_u32(smem);
  const uint32_t part_ready = bar_base + 8u * (uint32_t)(2 * kSplitMaxStages);
  const uint32_t recv_free = part_ready + 8u;
  auto full_bar = [&](int s) { return bar_base + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (uint32_t)(kSplitMaxStages + s); };
  const int n = p.st.n;
  const int ER = p.ER;
  if (tid < NS) {
    mbar_init(full_bar(tid), 1);
    mbar_init(empty_bar(tid), kSplitWarps);
    if (tid == 0) {
      mbar_init(part_ready, 1);
      mbar_init(recv_free, (uint32_t)C);
      *abort_flag = 0;
    }
    mbar_fence_init();
  }
  if (tid >= 32 && tid < 32 + B200_LORA_MAX_SLICES) {  // expand rows of this CTA, per slice
    const int s = tid - 32;
    const int out = s < n ? p.st.out[s] : 0;
    const int lo = min(c * p.oc[s], out);
    const int en = min(lo + p.oc[s], out) - lo;
    tab[s] = lo;
    tab[4 + s] = en;
    tab[8 + s] = (en + ER - 1) >> p.er_shift;
    tab[12 + s] = (s < n ? p.st.col[s] : 0) + lo;  // first y column of this CTA's rows of slice s
  }
  if (tid == kSplitConsumers)
    for (int s = 0; s < n; ++s) tma_prefetch_desc(&maps.a[s]);

  // uniform over the cluster: all CTAs of a bucket leave together
  if (slot < 0 || slot >= p.S || cnt <= 0 || start < 0 || start > p.T - cnt) return;
  int rank = p.r_max;
  if (p.rank_per_slot != nullptr) rank = min(max(p.rank_per_slot[slot], 0), p.r_max);
  const int r_eff = min(p.r_max, (rank + 31) & ~31);
  if (r_eff == 0) return;
  const float sc = p.scaling * (p.scale_per_slot != nullptr ? p.scale_per_slot[slot] : 1.0f);
  B200_TRACE_POINT(1)

  const int in_dim = p.in_dim;
  const int Kc = p.Kc, BC = p.BC, nchunk = p.nchunk;
  const int k_lo = c * Kc;
  const int nrb = r_eff >> 5;       // 32-row boxes per slice
  const int Qeff = n * r_eff;       // stacked rank rows
  const int npass = (cnt + 15) >> 4;

  __syncthreads();  // barriers and the row table are set up
  B200_TRACE_POINT(2)
  int tiles_exp = 0;
  for (int s = 0; s < n; ++s) tiles_exp += tab[8 + s];
  // Start-up cluster barrier: once it completes every CTA of the cluster has initialised its
  // barriers. Consumers wait on it before their first remote store, the producer before it exits.
  cluster_arrive();

  const int er_shift = p.er_shift;
  // next expand tile of this CTA in (slice, tile) order; the caller knows one is left
  auto next_tile = [&](int& cs, int& cet, int& s_out, int& r0_out) {
    while (cs < B200_LORA_MAX_SLICES - 1 && cet >= tab[8 + cs]) { ++cs; cet = 0; }
    s_out = cs;
    r0_out = cet << er_shift;
    ++cet;
  };

  if (warp == kSplitWarps) {
    // =========================== producer warp ===========================
    if (lane == 0) {
      int stage = 0, round = 0, issued = 0;
      auto acquire = [&]() -> uint32_t {
        if (round > 0) mbar_wait_bounded(empty_bar(stage), (uint32_t)((round & 1) ^ 1), abort_flag);
        return ring_base + (uint32_t)stage * (uint32_t)p.stage_bytes;
      };
      auto advance = [&]() {
        if (++stage == NS) { stage = 0; ++round; }
        if (++issued == NS) { B200_TRACE_PRODUCER(3) }
      };
      for (int pass = 0; pass < npass; ++pass) {
        // lora_A boxes: column chunk outer, (slice, 32-row box) inner -- the order the consumers use
        for (int j = 0; j < nchunk; ++j)
          for (int s = 0; s < n; ++s)
            for (int rb = 0; rb < nrb; ++rb) {
              const uint32_t dst = acquire();
              const uint32_t fb = full_bar(stage);
              mbar_arrive_expect_tx(fb, (uint32_t)p.a_stage_bytes);
              tma_load_2d(dst, &maps.a[s], k_lo + j * BC, slot * p.r_max + rb * kSplitBoxRows, fb);
              advance();
            }
        int cs = 0, cet = 0;
        for (int e = 0; e < tiles_exp; ++e) {
          int s, r0;
          next_tile(cs, cet, s, r0);
          const int nrows = min(ER, tab[4 + s] - r0);
          const uint32_t dst = acquire();
          const uint32_t fb = full_bar(stage);
          const uint32_t bytes = (uint32_t)nrows * (uint32_t)p.r_max * 2u;
          mbar_arrive_expect_tx(fb, bytes);
          const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(p.st.b[s]) +
                                     ((int64_t)slot * p.st.out[s] + tab[s] + r0) * p.r_max;
          bulk_g2s(dst, src, bytes, fb);
          advance();
        }
      }
    }
    __syncwarp();
    cluster_wait();
    return;
  }

  // ============================= consumer warps =============================
  // Everything that does not depend on x or y happens before the wait: token rows of the first
  // pass (index metadata), the start-up cluster barrier, arming the receive barrier, and an L2
  // prefetch of this CTA's activation and output columns (never into L1: a prefetch cannot create
  // stale data, L2 being the point of coherence).
  int tok0_lo = -1, tok0_hi = -1;
  if (g < cnt) tok0_lo = p.sorted_idx[start + g];
  if (g + 8 < cnt) tok0_hi = p.sorted_idx[start + g + 8];
  if (tok0_lo >= p.T) tok0_lo = -1;
  if (tok0_hi >= p.T) tok0_hi = -1;
  if (tid == 0) mbar_arrive_expect_tx(part_ready, (uint32_t)(C * 16 * Qeff * 4));
  const int G = n * nrb;  // 32-row boxes per column chunk (<= kSplitMaxGroups)
  if (p.use_pdl) {
    for (int kc = warp * 32 + t * 8; kc < Kc; kc += kSplitWarps * 32) {
      if (k_lo + kc < in_dim) {
        if (tok0_lo >= 0) prefetch_l2(p.x + (int64_t)tok0_lo * p.x_ld + k_lo + kc);
        if (tok0_hi >= 0) prefetch_l2(p.x + (int64_t)tok0_hi * p.x_ld + k_lo + kc);
      }
    }
    for (int s = 0; s < n; ++s) {
      const int en = tab[4 + s], cb = p.st.col[s] + tab[s];
      for (int r = warp * 32 + t * 8; r < en; r += kSplitWarps * 32) {
        if (tok0_lo >= 0) prefetch_l2(p.y + (int64_t)tok0_lo * p.y_ld + cb + r);
        if (tok0_hi >= 0) prefetch_l2(p.y + (int64_t)tok0_hi * p.y_ld + cb + r);
      }
    }
  }
  // Launch parameters live in constant memory that is cold for every new launch: whatever the code
  // after the wait needs is read here and pinned in registers, so that no constant-cache miss sits
  // on the critical path.
  uint32_t xs_base = smem_u32(smem + p.off_x), ys_base = smem_u32(smem + p.off_y);
  uint32_t recv_base = smem_u32(smem + p.off_recv), tmp_base = smem_u32(smem + p.off_tmp);
  uint32_t pitchB = (uint32_t)p.r_max * 2u, pitchA = (uint32_t)BC * 2u;
  uint32_t pitchX = (uint32_t)p.pitchX, pitchT = (uint32_t)p.pitchT, stage_bytes = (uint32_t)p.stage_bytes;
  int pitchP = p.pitchP, kblocks = r_eff >> 5, t_rows = p.T;
  const __nv_bfloat16* x_ptr = p.x;
  __nv_bfloat16* y_ptr = p.y;
  int64_t x_ld = p.x_ld, y_ld = p.y_ld;
  const int32_t* sorted_ptr = p.sorted_idx;
  asm volatile("" : "+r"(xs_base), "+r"(ys_base), "+r"(recv_base), "+r"(tmp_base), "+r"(pitchB), "+r"(pitchA));
  asm volatile("" : "+r"(pitchX), "+r"(pitchT), "+r"(stage_bytes), "+r"(pitchP), "+r"(kblocks), "+r"(t_rows));
  asm volatile("" : "+l"(x_ptr), "+l"(y_ptr), "+l"(x_ld), "+l"(y_ld), "+l"(sorted_ptr));
  int c_stage = 0, c_round = 0;
  auto advance = [&]() {
    if (++c_stage == NS) { c_stage = 0; ++c_round; }
  };
  cluster_wait();  // start-up barrier: peers run and their barriers are initialised
  if (p.use_pdl) griddep_wait();  // x and y of this launch are final from here on
  B200_TRACE_POINT(4)

  for (int pass = 0; pass < npass; ++pass) {
    int tok_lo = tok0_lo, tok_hi = tok0_hi;
    if (pass > 0) {
      tok_lo = tok_hi = -1;
      if (pass * 16 + g < cnt) tok_lo = sorted_ptr[start + pass * 16 + g];
      if (pass * 16 + g + 8 < cnt) tok_hi = sorted_ptr[start + pass * 16 + g + 8];
      if (tok_lo >= t_rows) tok_lo = -1;
      if (tok_hi >= t_rows) tok_hi = -1;
      if (tid == 0) mbar_arrive_expect_tx(part_ready, (uint32_t)(C * 16 * Qeff * 4));
    }

    // ---- stage x[16 tokens, Kc] (warp w copies token rows 4w..4w+3); absent rows / columns are zero.
    // Row r's token index sits in lane 4*(r%8) of this warp (tok_lo for r < 8, tok_hi above).
    // (plain loads into registers, then shared-memory stores: their issue does not serialise the way
    //  16-byte cp.async copies of rows nobody on this SM has touched do)
    int row_tok[4];  // the shuffles run with all 32 lanes, outside the lane-dependent column loop
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = warp * 4 + i;
      row_tok[i] = __shfl_sync(0xffffffffu, r < 8 ? tok_lo : tok_hi, (r & 7) * 4);
    }
    for (int k8 = lane * 8; k8 < Kc; k8 += 256) {
      uint4 xv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        xv[i] = make_uint4(0, 0, 0, 0);
        if (row_tok[i] >= 0 && k_lo + k8 < in_dim) xv[i] = ldg128(x_ptr + (int64_t)row_tok[i] * x_ld + k_lo + k8);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t dst = xs_base + (uint32_t)(warp * 4 + i) * pitchX + (uint32_t)k8 * 2u;
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(xv[i].x), "r"(xv[i].y), "r"(xv[i].z), "r"(xv[i].w) : "memory");
      }
    }
    cp_async_commit();  // (empty group: keeps the group count of the y slots below)
    if (pass == 0) { B200_TRACE_POINT(24) }

    // ---- request y of the first expand tiles (per-thread staging slots)
    int ycs = 0, yet = 0, yleft = tiles_exp;
    auto y_issue = [&](int d) {
      if (yleft > 0) {
        --yleft;
        int s, r0;
        next_tile(ycs, yet, s, r0);
        const int nrows = min(ER, tab[4 + s] - r0);
        const int col = tab[12 + s] + r0;
#pragma unroll
        for (int bi = 0; bi < 2; ++bi) {
          const int rb = (warp + kSplitWarps * bi) * 32;
          if (rb + 8 * t < nrows) {
            const uint32_t dst = ys_base + (uint32_t)((((d * 2 + bi) * 2) * kSplitConsumers + tid) * 16);
            if (tok_lo >= 0) cp_async16(dst, y_ptr + (int64_t)tok_lo * y_ld + col + rb + 8 * t);
            if (tok_hi >= 0) cp_async16(dst + kSplitConsumers * 16, y_ptr + (int64_t)tok_hi * y_ld + col + rb + 8 * t);
          }
        }
      }
      cp_async_commit();  // one group per slot, possibly empty: keeps the group count fixed
    };
#pragma unroll
    for (int d = 0; d < kSplitYDepth; ++d) y_issue(d);

    if (pass == 0) { B200_TRACE_POINT(25) }
    cp_async_wait<kSplitYDepth>();            // the x group (committed first) has landed
    if (pass == 0) { B200_TRACE_POINT(26) }
    named_bar_sync(1, kSplitConsumers);       // ... for every consumer thread
    if (pass == 0) { B200_TRACE_POINT(5) }
    // peers have read the partial sums of the previous pass out of their receive buffers
    if (pass > 0) mbar_wait_bounded_acquire_cluster(recv_free, (uint32_t)((pass - 1) & 1), abort_flag);

    // ===== shrink: partial[16 tok, 8 rows of this warp] over this CTA's columns, per 32-row box =====
    const uint32_t xlo_base = xs_base + (uint32_t)g * pitchX + (uint32_t)t * 16u;
    const uint32_t xhi_base = xlo_base + 8u * pitchX;
    // (tok g | g+8, stacked rows q, q+1) of this CTA's column range -> every CTA of the cluster
    auto send = [&](int grp, const float (&a)[4], const float (&b)[4]) {
      const int q = grp * 32 + 8 * warp + 2 * t;  // boxes are stacked in (slice, row box) order
      const uint32_t dlo = recv_base + (uint32_t)(((c * 16 + g) * pitchP + q) * 4);
      const uint32_t dhi = dlo + (uint32_t)(8 * pitchP * 4);
      for (int rc = 0; rc < C; ++rc) {
        const uint32_t rbar = mapa_shared(part_ready, (uint32_t)rc);
        st_async_f32x2(mapa_shared(dlo, (uint32_t)rc), a[0] + b[0], a[1] + b[1], rbar);
        st_async_f32x2(mapa_shared(dhi, (uint32_t)rc), a[2] + b[2], a[3] + b[3], rbar);
      }
    };
    {
      float acc[kSplitMaxGroups][4], acc2[kSplitMaxGroups][4];
#pragma unroll
      for (int grp = 0; grp < kSplitMaxGroups; ++grp)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[grp][i] = acc2[grp][i] = 0.f;
      for (int j = 0; j < nchunk; ++j) {
        // activation fragments of this column chunk, kept in registers for all boxes of the chunk
        uint4 xlo[kSplitBoxCols / 32], xhi[kSplitBoxCols / 32];
#pragma unroll
        for (int blk = 0; blk < kSplitBoxCols / 32; ++blk) {
          const int kl = j * BC + blk * 32;  // column inside this CTA's range
          xlo[blk] = xhi[blk] = make_uint4(0, 0, 0, 0);
          if (blk * 32 < BC && kl < Kc) {
            xlo[blk] = lds128(xlo_base + (uint32_t)kl * 2u);
            xhi[blk] = lds128(xhi_base + (uint32_t)kl * 2u);
          }
        }
#pragma unroll
        for (int grp = 0; grp < kSplitMaxGroups; ++grp) {
          if (grp < G) {
            mbar_wait_bounded(full_bar(c_stage), (uint32_t)(c_round & 1), abort_flag);
            const uint32_t wbase = ring_base + (uint32_t)c_stage * stage_bytes +
                                   (uint32_t)(8 * warp + g) * pitchA + (uint32_t)t * 16u;
            uint4 w[kSplitBoxCols / 32];
#pragma unroll
            for (int blk = 0; blk < kSplitBoxCols / 32; ++blk) {
              w[blk] = make_uint4(0, 0, 0, 0);
              if (blk * 32 < BC) w[blk] = lds128(wbase + (uint32_t)blk * 64u);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(c_stage));  // the box is in registers now
            advance();
#pragma unroll
            for (int blk = 0; blk < kSplitBoxCols / 32; ++blk) {
              mma_bf16_16816(acc[grp], xlo[blk].x, xhi[blk].x, xlo[blk].y, xhi[blk].y, w[blk].x, w[blk].y);
              mma_bf16_16816(acc2[grp], xlo[blk].z, xhi[blk].z, xlo[blk].w, xhi[blk].w, w[blk].z, w[blk].w);
            }
            if (j == nchunk - 1) send(grp, acc[grp], acc2[grp]);
            if (pass == 0 && grp == 0 && j == 0) { B200_TRACE_POINT(27) }
          }
        }
      }
    }
    if (pass == 0) { B200_TRACE_POINT(6) }

    // ===== add the C partials, scale, round to bf16 once =====
    mbar_wait_bounded_acquire_cluster(part_ready, (uint32_t)(pass & 1), abort_flag);
    if (pass == 0) { B200_TRACE_POINT(7) }
    {
      const int tok = tid >> 3;
      for (int pr = tid & 7; pr < (Qeff >> 1); pr += 8) {
        float2 v[8];
#pragma unroll
        for (int rc = 0; rc < 8; ++rc) {
          v[rc] = make_float2(0.f, 0.f);
          if (rc < C) v[rc] = lds_f32x2(recv_base + (uint32_t)(((rc * 16 + tok) * pitchP + 2 * pr) * 4));
        }
        const float s0 = ((v[0].x + v[1].x) + (v[2].x + v[3].x)) + ((v[4].x + v[5].x) + (v[6].x + v[7].x));
        const float s1 = ((v[0].y + v[1].y) + (v[2].y + v[3].y)) + ((v[4].y + v[5].y) + (v[6].y + v[7].y));
        sts32(tmp_base + (uint32_t)tok * pitchT + (uint32_t)pr * 4u, pack_bf16x2(s0 * sc, s1 * sc));
      }
    }
    if (pass == 0) { B200_TRACE_POINT(28) }
    named_bar_sync(1, kSplitConsumers);
    if (pass + 1 < npass && tid < C) mbar_arrive_remote_release(mapa_shared(recv_free, (uint32_t)tid));
    if (pass == 0) { B200_TRACE_POINT(8) }

    // ===== expand: y[tok, cols] += tmp[16 tok, r] . B_rows^T =====
    const uint32_t tmp_lo = tmp_base + (uint32_t)g * pitchT + (uint32_t)t * 16u;
    const uint32_t tmp_hi = tmp_lo + 8u * pitchT;
    int ccs = 0, cet = 0;
    for (int e = 0; e < tiles_exp; ++e) {
      int s_cur, r0;
      next_tile(ccs, cet, s_cur, r0);
      const int nrows = min(ER, tab[4 + s_cur] - r0);
      const int col = tab[12 + s_cur] + r0;
      const int d_slot = e % kSplitYDepth;
      mbar_wait_bounded(full_bar(c_stage), (uint32_t)(c_round & 1), abort_flag);
      if (pass == 0 && e < 1) { B200_TRACE_POINT(12 + 4 * e) }
      const uint32_t sbase = ring_base + (uint32_t)c_stage * stage_bytes;
      // this warp's (up to) two 32-row blocks of the tile, interleaved: 8 independent accumulators
      float d[2][4][4];
#pragma unroll
      for (int bi = 0; bi < 2; ++bi)
#pragma unroll
        for (int j = 0; j < 4; ++j) d[bi][j][0] = d[bi][j][1] = d[bi][j][2] = d[bi][j][3] = 0.f;
      for (int kb = 0; kb < kblocks; ++kb) {
        const uint32_t koff = (uint32_t)(s_cur * r_eff + kb * 32) * 2u;
        const uint4 alo = lds128(tmp_lo + koff);
        const uint4 ahi = lds128(tmp_hi + koff);
        uint4 w[2][4];
#pragma unroll
        for (int bi = 0; bi < 2; ++bi) {
          const int rb = (warp + kSplitWarps * bi) * 32;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            // MMA column n of tile j reads slab row 8*(n/2) + 2j + (n%2): thread (g,t) then owns
            // 8 consecutive output columns 8t..8t+7 of the block.
            const int prow = rb + 8 * (g >> 1) + 2 * j + (g & 1);
            w[bi][j] = make_uint4(0, 0, 0, 0);
            if (rb < nrows) w[bi][j] = lds128(sbase + (uint32_t)prow * pitchB + (uint32_t)(kb * 32 + t * 8) * 2u);
          }
        }
#pragma unroll
        for (int bi = 0; bi < 2; ++bi)
#pragma unroll
          for (int j = 0; j < 4; ++j) mma_bf16_16816(d[bi][j], alo.x, ahi.x, alo.y, ahi.y, w[bi][j].x, w[bi][j].y);
#pragma unroll
        for (int bi = 0; bi < 2; ++bi)
#pragma unroll
          for (int j = 0; j < 4; ++j) mma_bf16_16816(d[bi][j], alo.z, ahi.z, alo.w, ahi.w, w[bi][j].z, w[bi][j].w);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(c_stage));  // the tile is in registers now
      advance();
      if (pass == 0 && e < 1) { B200_TRACE_POINT(13 + 4 * e) }
      cp_async_wait<kSplitYDepth - 1>();  // y of tile e (this thread's own copies) is in its slot
#pragma unroll
      for (int bi = 0; bi < 2; ++bi) {
        const int rb = (warp + kSplitWarps * bi) * 32;
        if (rb + 8 * t < nrows) {
          const int cc = col + rb + 8 * t;
          const uint32_t src = ys_base + (uint32_t)((((d_slot * 2 + bi) * 2) * kSplitConsumers + tid) * 16);
          if (tok_lo >= 0) {
            uint4 v = lds128(src);
            v.x = add_bf16x2(v.x, d[bi][0][0], d[bi][0][1]);
            v.y = add_bf16x2(v.y, d[bi][1][0], d[bi][1][1]);
            v.z = add_bf16x2(v.z, d[bi][2][0], d[bi][2][1]);
            v.w = add_bf16x2(v.w, d[bi][3][0], d[bi][3][1]);
            stg128(y_ptr + (int64_t)tok_lo * y_ld + cc, v);
          }
          if (tok_hi >= 0) {
            uint4 v = lds128(src + kSplitConsumers * 16);
            v.x = add_bf16x2(v.x, d[bi][0][2], d[bi][0][3]);
            v.y = add_bf16x2(v.y, d[bi][1][2], d[bi][1][3]);
            v.z = add_bf16x2(v.z, d[bi][2][2], d[bi][2][3]);
            v.w = add_bf16x2(v.w, d[bi][3][2], d[bi][3][3]);
            stg128(y_ptr + (int64_t)tok_hi * y_ld + cc, v);
          }
        }
      }
      y_issue(d_slot);  // the slot is free again: request tile e + depth into it
      if (pass == 0 && e < 1) { B200_TRACE_POINT(14 + 4 * e) }
    }
    cp_async_wait<0>();
    if (pass == 0) { B200_TRACE_POINT(10) }
  }
  B200_TRACE_POINT(11)
  if (tid == 0 && *abort_flag != 0) atomicOr(&g_b200_status, kStatusWaitGaveUp);
}

// ------------------------------------------------------------------ host side
// 2-D bf16 row-major matrix [rows, cols] with row pitch `ld` elements, box = box_rows x box_cols,
// rows of a box dense in shared memory (no swizzle).
inline int make_tmap_2d_plain(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                              uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return fail(B200_LORA_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200_LORA_ECUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return B200_LORA_OK;
}

struct BgmvSplitOptions {
  int smem_kb = 0;  // cap of dynamic shared memory per CTA in KB (0 = default: two CTAs per SM)
};
inline BgmvSplitOptions& bgmv_split_options() {
  static BgmvSplitOptions o;
  return o;
}

// Fills `pp` with the tiling for this problem; false (and a reason) when this kernel cannot run it.
inline bool bgmv_split_plan(const BgmvProblem& b, BgmvSplitParams* pp, const char** why) {
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
  if (st.n * (b.r_max / 32) > kSplitMaxGroups) { *why = "n_slices * r_max / 32 exceeds the accumulator groups"; return false; }
  if ((int64_t)b.S * b.r_max > (1ll << 30)) { *why = "slab too tall for a tensor map"; return false; }

  const int Q = st.n * b.r_max;
  int C0 = bgmv_options().cluster;
  if (C0 != 1 && C0 != 2 && C0 != 4 && C0 != 8) {
    const int busy = std::min(b.n_buckets, std::max(b.T, 1));  // buckets that can hold tokens
    C0 = busy <= 37 ? 4 : (busy <= 74 ? 2 : 1);
  }
  const int cap0 = std::min(kBgmvSmemMax, (bgmv_split_options().smem_kb > 0 ? bgmv_split_options().smem_kb
                                                                           : kSplitDefaultSmemKb) * 1024);
  BgmvSplitParams p;
  p.y = static_cast<__nv_bfloat16*>(b.y); p.y_ld = b.y_ld;
  p.x = static_cast<const __nv_bfloat16*>(b.x); p.x_ld = b.x_ld;
  p.T = b.T; p.in_dim = b.in_dim; p.S = b.S; p.r_max = b.r_max; p.st = st;
  p.rank_per_slot = b.rank_per_slot; p.scale_per_slot = b.scale_per_slot;
  p.sorted_idx = b.sorted_idx; p.slot_ids = b.slot_ids; p.counts = b.counts; p.offsets = b.offsets;
  p.n_buckets = b.n_buckets; p.scaling = b.scaling;
  p.use_pdl = bgmv_options().pdl ? 1 : 0;
  p.ER = std::max(32, std::min(256, floor_pow2(16384 / (b.r_max * 2))));
  p.er_shift = log2_exact(p.ER);
  p.BC = std::min(kSplitBoxCols, b.in_dim);
  p.a_stage_bytes = p.BC * kSplitBoxRows * 2;
  p.stage_bytes = round_up_i(std::max(p.a_stage_bytes, p.ER * b.r_max * 2), 128);
  p.pitchT = round_up_i(Q * 2, 128) + 64;
  p.pitchP = Q;
  const int tmp_bytes = round_up_i(kBgmvTok * p.pitchT, 128);
  // A smaller cluster keeps more columns per CTA: widen the cluster until the buffers fit, first
  // under the cap that lets two CTAs share an SM, then with all of an SM's shared memory.
  for (int cap = cap0; cap <= kBgmvSmemMax; cap = (cap < kBgmvSmemMax ? kBgmvSmemMax : kBgmvSmemMax + 1))
  for (int C = C0; C <= 8; C *= 2) {
    p.c_shift = log2_exact(C);
    p.Kc = round_up_i(ceil_div_i(b.in_dim, C), 32);
    p.nchunk = ceil_div_i(p.Kc, p.BC);
    p.pitchX = round_up_i(p.Kc * 2, 128) + 64;
    int tiles_exp = 0;
    for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) p.oc[s] = 0;
    for (int s = 0; s < st.n; ++s) {
      p.oc[s] = round_up_i(ceil_div_i(st.out[s], C), 32);
      tiles_exp += ceil_div_i(p.oc[s], p.ER);
    }
    const int tiles = st.n * (b.r_max / 32) * p.nchunk + tiles_exp;
    const int x_bytes = round_up_i(kBgmvTok * p.pitchX, 128);
    const int y_bytes = std::min(kSplitYDepth, std::max(tiles_exp, 1)) * kSplitYSlotBytes;
    const int recv_bytes = round_up_i(C * kBgmvTok * p.pitchP * 4, 128);
    const int bar_bytes = 512;
    const int fixed = x_bytes + y_bytes + recv_bytes + tmp_bytes + bar_bytes;
    int NS = std::min(std::min(tiles, kSplitMaxStages), (cap - fixed) / p.stage_bytes);
    if (fixed >= cap || NS < 2) continue;
    p.NS = NS;
    p.off_x = NS * p.stage_bytes;
    p.off_y = p.off_x + x_bytes;
    p.off_recv = p.off_y + y_bytes;
    p.off_tmp = p.off_recv + recv_bytes;
    p.off_bar = p.off_tmp + tmp_bytes;
    if (pp != nullptr) *pp = p;
    return true;
  }
  *why = "buffers of the column-split kernel do not fit the shared-memory cap";
  return false;
}

inline bool bgmv_split_supported(const BgmvProblem& b, const char** why) { return bgmv_split_plan(b, nullptr, why); }

inline int bgmv_split_launch(const BgmvProblem& b, cudaStream_t stream) {
  BgmvSplitParams p;
  const char* why = nullptr;
  if (!bgmv_split_plan(b, &p, &why)) return fail(B200_LORA_EUNSUPPORTED, "column-split decode kernel: %s", why);
  BgmvSplitMaps maps;
  for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) {
    const int src = s < p.st.n ? s : 0;  // unused entries repeat a valid map
    if (int rc = make_tmap_2d_plain(&maps.a[s], p.st.a[src], (uint64_t)p.S * p.r_max, (uint64_t)p.in_dim,
                                    (uint64_t)p.in_dim, kSplitBoxRows, (uint32_t)p.BC))
      return rc;
  }
  const size_t smem = (size_t)p.off_bar + 512;
  static thread_local int configured_device = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(bgmv_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBgmvSmemMax);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(bgmv_split_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                               cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return fail(B200_LORA_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured_device = dev;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1u << p.c_shift, (unsigned)p.n_buckets, 1);
  cfg.blockDim = dim3(kSplitThreads, 1, 1);
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
  cudaError_t e = cudaLaunchKernelEx(&cfg, bgmv_split_kernel, p, maps);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(B200_LORA_ECUDA, "bgmv_split_kernel launch: %s", cudaGetErrorString(e));
  }
  return B200_LORA_OK;
}

}  // namespace b200lora
