// Device-side build of the per-step LoRA index metadata from token_to_slot: a stable counting
// sort of the token rows by adapter slot, the tokens per slot and the bucket start offsets, in
// the three conventions the reference produces on the host with Python loops over the tokens
// (nanovllm_voxcpm/engine/lora_manager.py:77-111, engine/model_runner.py:774-797,
// lora_ops/triton_ops/lora_kernel_metadata.py:47-67). One CTA, one launch, no host work, and the
// arrays it writes are identical bit for bit to the host builders' (integer work).
//
//   GRAPH   fixed buckets [-1, 0, .., S-1]: counts[0] = 0, counts[s+1] = rows of slot s,
//           offsets[0..S+1] = running sum, sorted_idx[0 .. rows with an adapter) (the tail of the
//           buffer keeps whatever it held, as in the reference's graph buffers)
//   KERNEL  compact buckets of the ids that occur, ascending, the -1 bucket first WITH its rows;
//           unused ids = -1, unused counts = 0, offsets[1..k] = running sum and 0 elsewhere;
//           sorted_idx holds all T rows
//   EAGER   compact buckets of the slots >= 0 that occur; rows without adapter are absent
// info[0] = buckets in use (k), info[1] = rows with an adapter, info[2] = rows whose slot id was
// outside [-1, S) (they are treated as "no adapter").
#pragma once

#include <cub/block/block_radix_sort.cuh>
#include <cub/block/block_scan.cuh>

#include "common.cuh"

namespace b200lora {

constexpr int kMetaThreads = 1024;
constexpr int kMetaMaxSlots = 4095;     // buckets (S + 1) <= 4096: 4 per thread
constexpr int kMetaMaxTokens = 16384;   // 16 keys per thread
constexpr int kMetaBucketsPerThread = 4;

template <int ITEMS>
__global__ void __launch_bounds__(kMetaThreads, 1)
build_metadata_kernel(const int32_t* __restrict__ token_to_slot, int T, int S, int mode, int32_t* __restrict__ sorted_idx,
                      int32_t* __restrict__ slot_ids, int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                      int32_t* __restrict__ info) {
  using Sort = cub::BlockRadixSort<uint32_t, kMetaThreads, ITEMS>;
  using Scan = cub::BlockScan<int, kMetaThreads>;
  extern __shared__ __align__(16) uint8_t meta_smem[];
  typename Sort::TempStorage& sort_tmp = *reinterpret_cast<typename Sort::TempStorage*>(meta_smem);
  __shared__ typename Scan::TempStorage scan_tmp;
  __shared__ int hist[kMetaMaxSlots + 1];   // rows per bucket, bucket = slot + 1
  __shared__ int bad_rows;
  const int tid = threadIdx.x;
  const int nb = S + 1;

  for (int b = tid; b < nb; b += kMetaThreads) hist[b] = 0;
  if (tid == 0) bad_rows = 0;
  __syncthreads();

  // keys: bucket in the high half, row in the low 16 bits; ascending key order is the stable
  // order (rows of one slot stay in their original order); padding keys sort last
  uint32_t keys[ITEMS];
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int t = tid * ITEMS + k;
    keys[k] = 0xffffffffu;
    if (t < T) {
      int slot = token_to_slot[t];
      if (slot < -1 || slot >= S) { slot = -1; atomicAdd(&bad_rows, 1); }
      atomicAdd(&hist[slot + 1], 1);
      keys[k] = ((uint32_t)(slot + 1) << 16) | (uint32_t)t;
    }
  }
  __syncthreads();
  const int none_rows = hist[0];
  // KERNEL convention with no adapter row at all: the host builder returns before it fills anything
  // (ids -1, counts 0, offsets 0, sorted rows untouched)
  const bool nothing = mode == 1 && none_rows == T;
  int end_bit = 17;
  while ((1 << (end_bit - 16)) < nb + 1 && end_bit < 32) ++end_bit;
  Sort(sort_tmp).Sort(keys, 0, end_bit);
  // position of a key in the sorted order = tid * ITEMS + k (blocked arrangement)
  const int skip = mode == 1 ? 0 : none_rows;  // GRAPH / EAGER leave rows without adapter out
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int pos = tid * ITEMS + k;
    if (keys[k] != 0xffffffffu && pos >= skip && !nothing) sorted_idx[pos - skip] = (int32_t)(keys[k] & 0xffffu);
  }

  // buckets: this thread owns buckets [4 tid, 4 tid + 4)
  int cnt[kMetaBucketsPerThread], used = 0, rows = 0;
#pragma unroll
  for (int i = 0; i < kMetaBucketsPerThread; ++i) {
    const int b = tid * kMetaBucketsPerThread + i;
    cnt[i] = b < nb ? hist[b] : 0;
    if ((b == 0 && mode != 1) || nothing) cnt[i] = 0;  // the -1 bucket counts only in KERNEL mode
    used += cnt[i] > 0;
    rows += cnt[i];
  }
  int used_before, rows_before, used_total, rows_total;
  Scan(scan_tmp).ExclusiveSum(used, used_before, used_total);
  __syncthreads();
  Scan(scan_tmp).ExclusiveSum(rows, rows_before, rows_total);
  if (mode == 0) {
#pragma unroll
    for (int i = 0; i < kMetaBucketsPerThread; ++i) {
      const int b = tid * kMetaBucketsPerThread + i;
      if (b < nb) {
        counts[b] = cnt[i];
        offsets[b] = rows_before;
        if (slot_ids != nullptr) slot_ids[b] = b - 1;
        rows_before += cnt[i];
        if (b == nb - 1) offsets[nb] = rows_before;
      }
    }
  } else {
    // unused tail first (disjoint from the entries written below: index >= used_total)
    for (int b = used_total + tid; b < nb; b += kMetaThreads) {
      slot_ids[b] = -1;
      counts[b] = 0;
    }
    for (int b = used_total + 1 + tid; b <= nb; b += kMetaThreads) offsets[b] = 0;
    if (tid == 0) offsets[0] = 0;
#pragma unroll
    for (int i = 0; i < kMetaBucketsPerThread; ++i) {
      const int b = tid * kMetaBucketsPerThread + i;
      if (b < nb && cnt[i] > 0) {
        slot_ids[used_before] = b - 1;
        counts[used_before] = cnt[i];
        rows_before += cnt[i];
        offsets[used_before + 1] = rows_before;
        ++used_before;
      }
    }
  }
  if (info != nullptr && tid == 0) {
    info[0] = mode == 0 ? nb : used_total;
    info[1] = T - none_rows;
    info[2] = bad_rows;
  }
}

template <int ITEMS>
inline int launch_build_metadata(const int32_t* tts, int T, int S, int mode, int32_t* sorted_idx, int32_t* slot_ids,
                                 int32_t* counts, int32_t* offsets, int32_t* info, cudaStream_t stream) {
  using Sort = cub::BlockRadixSort<uint32_t, kMetaThreads, ITEMS>;
  const size_t smem = sizeof(typename Sort::TempStorage);
  static thread_local int configured_device = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_device != dev) {  // sort scratch + the static histogram exceed the 48 KB default
    cudaError_t e = cudaFuncSetAttribute(build_metadata_kernel<ITEMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(B200_LORA_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    configured_device = dev;
  }
  build_metadata_kernel<ITEMS><<<1, kMetaThreads, smem, stream>>>(tts, T, S, mode, sorted_idx, slot_ids, counts, offsets, info);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_LORA_ECUDA, "build_metadata_kernel launch: %s", cudaGetErrorString(e));
  return B200_LORA_OK;
}

inline int build_metadata(const int32_t* tts, int T, int S, int mode, int32_t* sorted_idx, int32_t* slot_ids,
                          int32_t* counts, int32_t* offsets, int32_t* info, cudaStream_t stream) {
  if (T < 0 || T > kMetaMaxTokens) return fail(B200_LORA_EUNSUPPORTED, "metadata build: T=%d outside [0, %d]", T, kMetaMaxTokens);
  if (S < 1 || S > kMetaMaxSlots) return fail(B200_LORA_EUNSUPPORTED, "metadata build: S=%d outside [1, %d]", S, kMetaMaxSlots);
  if (mode < 0 || mode > 2) return fail(B200_LORA_EINVAL, "metadata build: unknown convention %d", mode);
  if (counts == nullptr || offsets == nullptr || (T > 0 && (tts == nullptr || sorted_idx == nullptr)))
    return fail(B200_LORA_EINVAL, "metadata build: null array");
  if (mode != 0 && slot_ids == nullptr) return fail(B200_LORA_EINVAL, "metadata build: this convention writes slot_ids");
  if (T <= 1024) return launch_build_metadata<1>(tts, T, S, mode, sorted_idx, slot_ids, counts, offsets, info, stream);
  if (T <= 4096) return launch_build_metadata<4>(tts, T, S, mode, sorted_idx, slot_ids, counts, offsets, info, stream);
  return launch_build_metadata<16>(tts, T, S, mode, sorted_idx, slot_ids, counts, offsets, info, stream);
}

}  // namespace b200lora
