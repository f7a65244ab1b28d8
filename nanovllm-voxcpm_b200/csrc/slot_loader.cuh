// Adapter admission in one launch: writes every slab region of one adapter slot from a packed
// staging buffer (zero padding beyond the effective rank, adapter scaling folded into lora_B) and
// the slot's rank / scaling entries of every module.
//
// The reference loads a slot module by module (nanovllm_voxcpm/engine/model_runner.py:389-420):
// per module one host->device copy per tensor, a zero_() of the slot and copies of the [:rank] rows /
// columns, B multiplied by the scaling first (nanovllm_voxcpm/layers/lora.py:395-417) - dozens of
// small launches per admission. Here the host packs one table of descriptors plus all payload
// tensors into ONE pinned buffer, copies it once, and this kernel does the rest. The values written
// are those of the reference: dst = round_to_slab_dtype(float(src) * scale) inside the payload's
// [rows_used, cols_used] corner, zero elsewhere.
#pragma once

#include "common.cuh"

namespace b200lora {

constexpr int kSlotLoadThreads = 256;
constexpr int kSlotLoadChunk = 8192;  // destination elements per CTA

// kind 0: padded 2-D copy into a slab's slot region; kind 1: int32 scalar; kind 2: floating scalar of dst_dtype
struct SlotLoadDesc {
  void* dst;             // slot region [dst_rows, dst_cols] (contiguous), or the scalar's address
  int64_t src_offset;    // byte offset of the payload inside the staging buffer (kind 0)
  int32_t kind;
  int32_t dst_rows, dst_cols;
  int32_t src_rows, src_cols, src_ld;  // corner that holds data, and the payload's row pitch (elements)
  int32_t src_dtype, dst_dtype;        // B200_LORA_BF16 / F16 / F32
  float scale;                         // kind 0: multiplier; kind 2: the value
  int32_t ivalue;                      // kind 1: the value
  int32_t pad_;
};
static_assert(sizeof(SlotLoadDesc) == 64, "descriptor layout is part of the host <-> device contract");

__device__ __forceinline__ float slot_load_src(const uint8_t* base, int dtype, int64_t idx) {
  if (dtype == B200_LORA_F32) return reinterpret_cast<const float*>(base)[idx];
  if (dtype == B200_LORA_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  return __half2float(reinterpret_cast<const __half*>(base)[idx]);
}

__global__ void __launch_bounds__(kSlotLoadThreads) slot_load_kernel(const SlotLoadDesc* __restrict__ table,
                                                                     const uint8_t* __restrict__ staging) {
  const SlotLoadDesc d = table[blockIdx.y];
  // descriptor sanity (bounds-checked build): kinds, dtypes, and the data corner inside both the slot region
  // and the payload's row pitch
  if (!B200_IN_BOUNDS(d.dst != nullptr && d.kind >= 0 && d.kind <= 2 && d.dst_dtype >= 0 && d.dst_dtype <= 2 &&
                      (d.kind != 0 || (d.src_dtype >= 0 && d.src_dtype <= 2 && d.dst_rows >= 0 && d.dst_cols >= 0 &&
                                       d.src_rows >= 0 && d.src_rows <= d.dst_rows && d.src_cols >= 0 &&
                                       d.src_cols <= d.dst_cols && d.src_cols <= d.src_ld && d.src_offset >= 0))))
    return;
  if (d.kind == 1) {
    if (blockIdx.x == 0 && threadIdx.x == 0) *static_cast<int32_t*>(d.dst) = d.ivalue;
    return;
  }
  if (d.kind == 2) {  // the scaling buffers take the module's floating dtype when a model is cast
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      if (d.dst_dtype == B200_LORA_BF16) *static_cast<__nv_bfloat16*>(d.dst) = __float2bfloat16_rn(d.scale);
      else if (d.dst_dtype == B200_LORA_F16) *static_cast<__half*>(d.dst) = __float2half_rn(d.scale);
      else *static_cast<float*>(d.dst) = d.scale;
    }
    return;
  }
  const int64_t total = (int64_t)d.dst_rows * d.dst_cols;
  const int64_t lo = (int64_t)blockIdx.x * kSlotLoadChunk;
  if (lo >= total) return;
  const int64_t hi = min(lo + (int64_t)kSlotLoadChunk, total);
  const uint8_t* src = staging + d.src_offset;
  for (int64_t i = lo + threadIdx.x; i < hi; i += kSlotLoadThreads) {
    const int row = (int)(i / d.dst_cols), col = (int)(i - (int64_t)row * d.dst_cols);
    float v = 0.f;
    if (row < d.src_rows && col < d.src_cols) {
      v = slot_load_src(src, d.src_dtype, (int64_t)row * d.src_ld + col) * d.scale;
      // the reference multiplies in the payload's own dtype before it copies into the slab
      if (d.src_dtype == B200_LORA_F16) v = __half2float(__float2half_rn(v));
      else if (d.src_dtype == B200_LORA_BF16) v = __bfloat162float(__float2bfloat16_rn(v));
    }
    if (d.dst_dtype == B200_LORA_BF16) static_cast<__nv_bfloat16*>(d.dst)[i] = __float2bfloat16_rn(v);
    else if (d.dst_dtype == B200_LORA_F16) static_cast<__half*>(d.dst)[i] = __float2half_rn(v);
    else static_cast<float*>(d.dst)[i] = v;
  }
}

// `staging`: device copy of the packed buffer, `n_desc` descriptors at its start; `max_elems`: the
// largest dst_rows * dst_cols among them (sizes the grid).
inline int slot_load_launch(const void* staging, int n_desc, int64_t max_elems, cudaStream_t stream) {
  if (n_desc < 0 || max_elems < 0) return fail(B200_LORA_EINVAL, "slot load: negative count");
  if (n_desc == 0) return B200_LORA_OK;
  if (staging == nullptr) return fail(B200_LORA_EINVAL, "slot load: null staging buffer");
  if (n_desc > 65535) return fail(B200_LORA_EUNSUPPORTED, "slot load: more than 65535 descriptors");
  const int64_t chunks = std::max<int64_t>(1, (max_elems + kSlotLoadChunk - 1) / kSlotLoadChunk);
  if (chunks > 0x7fffffff) return fail(B200_LORA_EUNSUPPORTED, "slot load: region too large");
  slot_load_kernel<<<dim3((unsigned)chunks, (unsigned)n_desc), kSlotLoadThreads, 0, stream>>>(
      static_cast<const SlotLoadDesc*>(staging), static_cast<const uint8_t*>(staging));
  return check_launch("slot_load_kernel");
}

}  // namespace b200lora
