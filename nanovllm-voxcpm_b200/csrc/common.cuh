// Shared host/device helpers for the multi-LoRA kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>

#include "../../include/b200_lora.h"

namespace b200lora {

// ---------------------------------------------------------------- host side
// Last error message of the calling thread, returned by lora_b200_last_error().
inline char* error_buffer() {
  static thread_local char buf[512] = "";
  return buf;
}

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_LORA_ECUDA, "%s: %s", what, cudaGetErrorString(e));
  return B200_LORA_OK;
}

inline size_t dtype_size(int dtype) { return dtype == B200_LORA_F32 ? 4 : 2; }

// Slice table passed by value to every kernel (<= 4 slices: q/k/v, gate/up, or 1).
struct SliceTable {
  const void* a[B200_LORA_MAX_SLICES];  // [S, r_max, in]
  const void* b[B200_LORA_MAX_SLICES];  // [S, out_s, r_max]
  int32_t out[B200_LORA_MAX_SLICES];    // width of the slice
  int32_t col[B200_LORA_MAX_SLICES];    // first y column of the slice
  int32_t n;
};

// --------------------------------------------------------------- device side
// Status word of the device (lora_b200_device_status): kernels never trap, they raise a bit and carry on.
constexpr int kStatusWaitGaveUp = 1;        // a bounded wait on an mbarrier ran out
constexpr int kStatusPeerWaitGaveUp = 2;    // a bounded wait on another rank's flag ran out
constexpr int kStatusBadSmemBase = 4;       // dynamic shared memory was not 1024-byte aligned
constexpr int kStatusBoundsViolation = 8;   // bounds-checked build only: an index left its array

__device__ int g_b200_status = 0;

// Bounds-checked build (-DB200_LORA_DEBUG_BOUNDS, lib/libb200lora_debug.so): every slot, row and column
// index that comes from caller-provided metadata, and every copy range derived from it, is checked before
// use; a violation raises kStatusBoundsViolation and the access is skipped. In the product build the checks
// compile to nothing. (The pool's memory checker is not available to this project; this build takes its place.)
#ifdef B200_LORA_DEBUG_BOUNDS
__device__ __noinline__ bool bounds_violation() {
  atomicOr(&g_b200_status, kStatusBoundsViolation);
  return false;
}
#define B200_IN_BOUNDS(cond) ((cond) ? true : b200lora::bounds_violation())
#else
#define B200_IN_BOUNDS(cond) true
#endif

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace b200lora
