// Thin inline-PTX wrappers (sm_100a): mbarrier, bulk async copies (TMA unit),
// thread-block clusters / distributed shared memory, programmatic dependent
// launch, warp-level bf16 MMA. Every blocking wait here is bounded.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200lora {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrive without release semantics: for "this stage may be refilled" signals, where the data read from
// the stage is already in registers. (A releasing arrive first waits for the thread's outstanding
// global stores and reductions, a round trip to the L2 per tile in an epilogue that writes y.)
__device__ __forceinline__ void mbar_arrive_relaxed(uint32_t bar) {
  asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrive on an mbarrier of another CTA of the cluster (address from mapa_shared); the
// release at cluster scope publishes this CTA's earlier distributed-shared-memory stores.
__device__ __forceinline__ void mbar_arrive_remote_release(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait_acquire_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Wait for `parity` of `bar`, giving up after kSpinLimit polls. A give-up raises
// *abort_flag (shared memory); once it is raised every later wait of the CTA
// returns at once, so control flow never depends on a barrier that cannot
// complete. Returns false when it gave up.
constexpr int kSpinLimit = 1 << 22;
// The polling loops live out of line: a wait whose barrier has already completed (the common case
// once the weights are resident) costs one try_wait at the call site, and the kernels' code stays
// small enough for the instruction cache.
__device__ __noinline__ bool mbar_spin_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (int it = 0; it < kSpinLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag != 0) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __noinline__ bool mbar_spin_bounded_acquire_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (int it = 0; it < kSpinLimit; ++it) {
    if (mbar_try_wait_acquire_cluster(bar, parity)) return true;
    if (*abort_flag != 0) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_spin_bounded(bar, parity, abort_flag);
}
__device__ __forceinline__ bool mbar_wait_bounded_acquire_cluster(uint32_t bar, uint32_t parity,
                                                                  volatile int* abort_flag) {
  if (mbar_try_wait_acquire_cluster(bar, parity)) return true;
  return mbar_spin_bounded_acquire_cluster(bar, parity, abort_flag);
}

// ---------------------------------------------------- bulk async copy (1-D)
// global -> shared, completion counted in bytes on an mbarrier. Addresses and
// size must be multiples of 16 bytes.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// L2 prefetch of a contiguous global range by the TMA unit (no shared memory, no completion
// to wait for); address and size multiples of 16 bytes.
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// Bulk (TMA unit) copies shared -> global, tracked in the issuing thread's bulk async-groups: plain
// store, and bf16 addition performed at the L2. Addresses and size multiples of 16 bytes.
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_reduce_add_bf16(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.bf16 [%0], [%1], %2;" ::"l"(dst), "r"(src_smem),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the thread's earlier bulk groups have finished reading shared memory / have completed
__device__ __forceinline__ void bulk_wait_all_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ------------------------------------------------------------------ cluster
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t local_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(cta_rank));
  return r;
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// 8-byte store into the shared memory of a CTA of the cluster that also counts its bytes on
// an mbarrier of that CTA (both addresses from mapa_shared): data and signal in one operation.
__device__ __forceinline__ void st_async_b32x2(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t cluster_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.b32 [%0], {%1, %2}, [%3];" ::"r"(cluster_addr),
               "r"(a), "r"(b), "r"(cluster_bar)
               : "memory");
}
__device__ __forceinline__ void st_async_f32x4(uint32_t cluster_addr, float4 v, uint32_t cluster_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(cluster_addr),
               "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "r"(cluster_bar)
               : "memory");
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}

// barrier among a subset of the CTA's warps (id 1..15, thread count a multiple of 32)
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ------------------------------------------ programmatic dependent launch
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ------------------------------------------------------------ loads / stores
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// 16-byte global load through the read-only path (data not written by this kernel)
__device__ __forceinline__ uint4 ldg128_nc(const void* gptr) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(gptr));
  return v;
}
__device__ __forceinline__ void prefetch_l2(const void* gptr) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(gptr));
}
__device__ __forceinline__ uint4 ldg128(const void* gptr) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(gptr) : "memory");
  return v;
}
__device__ __forceinline__ void stg128(void* gptr, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(gptr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// y[0..8) += d[0..8) (bf16, one 16-byte reduction performed at the L2; nothing comes back)
__device__ __forceinline__ void red_add_bf16x8(void* gptr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(gptr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// ------------------------------------------------- warp MMA, bf16 -> fp32
// D(16x8) += A(16x16, row) * B(16x8, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
// two packed bf16 + two fp32 deltas, rounded once
__device__ __forceinline__ uint32_t add_bf16x2(uint32_t y, float d0, float d1) {
  return pack_bf16x2(bf16_lo(y) + d0, bf16_hi(y) + d1);
}

}  // namespace b200lora
