// L2 prefetch of the adapter weights a step is about to use.
//
// In a decoder step every multi-LoRA launch follows a base GEMM of a library, which does not let the next
// kernel start early, so the launch's first HBM round trip (the slot's lora_A / lora_B rows, 0.1 - 1 MB per
// bucket) lies on the critical path of the step. This kernel, launched on a side stream one layer ahead,
// asks the memory system to bring the slot regions of the ACTIVE buckets into L2 (cp.async.bulk.prefetch.L2,
// a hint: nothing is written, nothing has to be waited for), so that the launches find them there.
#pragma once

#include "common.cuh"

namespace b200lora {

constexpr int kPrefetchMaxSlabs = 16;
constexpr int kPrefetchThreads = 128;
constexpr int kPrefetchChunk = 4096;  // bytes per prefetch request

struct PrefetchTable {
  const uint8_t* base[kPrefetchMaxSlabs];   // slab [S, ...]
  int64_t slot_stride[kPrefetchMaxSlabs];   // bytes from one slot's region to the next
  int64_t bytes[kPrefetchMaxSlabs];         // bytes of a slot's region to fetch (multiple of 16)
  int n;
};

__global__ void __launch_bounds__(kPrefetchThreads) prefetch_slabs_kernel(const PrefetchTable t,
                                                                          const int32_t* __restrict__ slot_ids,
                                                                          const int32_t* __restrict__ counts, int S) {
  const int slot = slot_ids[blockIdx.x];
  if (slot < 0 || slot >= S || (counts != nullptr && counts[blockIdx.x] <= 0)) return;
  const int j = blockIdx.y;
  const uint8_t* p = t.base[j] + (int64_t)slot * t.slot_stride[j];
  const int64_t total = t.bytes[j];
  for (int64_t off = (int64_t)threadIdx.x * kPrefetchChunk; off < total; off += (int64_t)kPrefetchThreads * kPrefetchChunk) {
    const uint32_t n = (uint32_t)min((int64_t)kPrefetchChunk, total - off) & ~15u;
    if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p + off), "r"(n) : "memory");
  }
}

inline int prefetch_slabs_launch(const void* const* slabs, const int64_t* slot_stride_bytes, const int64_t* bytes_per_slot,
                                 int n_slabs, const int32_t* slot_ids, const int32_t* counts, int n_buckets, int S,
                                 cudaStream_t stream) {
  if (n_slabs < 0 || n_buckets < 0 || S < 0) return fail(B200_LORA_EINVAL, "prefetch: negative count");
  if (n_slabs == 0 || n_buckets == 0) return B200_LORA_OK;
  if (n_slabs > kPrefetchMaxSlabs) return fail(B200_LORA_EUNSUPPORTED, "prefetch: more than %d slabs per call", kPrefetchMaxSlabs);
  if (slabs == nullptr || slot_stride_bytes == nullptr || bytes_per_slot == nullptr || slot_ids == nullptr)
    return fail(B200_LORA_EINVAL, "prefetch: null pointer");
  PrefetchTable t;
  t.n = n_slabs;
  for (int j = 0; j < n_slabs; ++j) {
    if (slabs[j] == nullptr || (reinterpret_cast<uintptr_t>(slabs[j]) & 15) || (slot_stride_bytes[j] & 15) || bytes_per_slot[j] < 0)
      return fail(B200_LORA_EINVAL, "prefetch: slab %d must be 16-byte aligned with a 16-byte multiple per slot", j);
    t.base[j] = static_cast<const uint8_t*>(slabs[j]);
    t.slot_stride[j] = slot_stride_bytes[j];
    t.bytes[j] = bytes_per_slot[j];
  }
  prefetch_slabs_kernel<<<dim3((unsigned)n_buckets, (unsigned)n_slabs), kPrefetchThreads, 0, stream>>>(t, slot_ids, counts, S);
  return check_launch("prefetch_slabs_kernel");
}

}  // namespace b200lora
