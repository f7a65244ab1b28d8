// Generic multi-LoRA kernels: one CTA per token, any dtype, shape and row stride.
// They are the correctness floor (fp16 / fp32 layers, tiny test shapes, odd ranks);
// the bf16 decode / prefill kernels in bgmv_fused.cuh and sgmv_tc.cuh carry the load.
#pragma once

#include "common.cuh"

namespace b200lora {

constexpr int kGenericThreads = 256;

// y[t, col_s + o] += sc * sum_j (x[t] . A_s[slot][j]) * B_s[slot][o][j]
// Follows the per-token formula of the reference's backends
// (nanovllm_voxcpm/lora.py:241-381; tests/unit/test_lora_layers.py:17-48).
template <typename T>
__global__ void __launch_bounds__(kGenericThreads)
generic_add_kernel(T* __restrict__ y, int64_t y_ld, const T* __restrict__ x, int64_t x_ld,
                   int in_dim, SliceTable st, int S, int r_max,
                   const int32_t* __restrict__ rank_per_slot,
                   const float* __restrict__ scale_per_slot,
                   const int32_t* __restrict__ token_to_slot, float scaling) {
  extern __shared__ float tmp[];  // [n, r_max]
  const int t = blockIdx.x;
  const int slot = token_to_slot[t];
  (void)B200_IN_BOUNDS(slot >= -1 && slot < S);
  if (slot < 0 || slot >= S) return;  // rows without an adapter are never touched
  int r = r_max;
  if (rank_per_slot != nullptr) r = min(max(rank_per_slot[slot], 0), r_max);
  if (r == 0) return;
  const float sc = scaling * (scale_per_slot != nullptr ? scale_per_slot[slot] : 1.0f);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const T* xr = x + (int64_t)t * x_ld;

  for (int q = warp; q < st.n * r; q += nwarps) {
    const int s = q / r, j = q - s * r;
    if (st.out[s] == 0) continue;
    const T* arow = static_cast<const T*>(st.a[s]) + ((int64_t)slot * r_max + j) * in_dim;
    float acc = 0.f;
    for (int k = lane; k < in_dim; k += 32) acc += to_float(xr[k]) * to_float(arow[k]);
    acc = warp_sum(acc);
    if (lane == 0) tmp[s * r_max + j] = acc * sc;
  }
  __syncthreads();

  for (int s = 0; s < st.n; ++s) {
    const int out = st.out[s];
    if (out == 0) continue;
    const T* b = static_cast<const T*>(st.b[s]) + (int64_t)slot * out * r_max;
    const float* ts = tmp + s * r_max;
    T* yr = y + (int64_t)t * y_ld + st.col[s];
    for (int o = threadIdx.x; o < out; o += blockDim.x) {
      const T* brow = b + (int64_t)o * r_max;
      float acc = 0.f;
      for (int j = 0; j < r; ++j) acc += ts[j] * to_float(brow[j]);
      yr[o] = from_float<T>(to_float(yr[o]) + acc);
    }
  }
}

// out[s, t, :] = scaling * x[t] . A_s[slot]^T, zero rows for slot < 0
// (nanovllm_voxcpm/lora_ops/triton_ops/lora_shrink_op.py:257-341).
template <typename T, typename TO>
__global__ void __launch_bounds__(kGenericThreads)
generic_shrink_kernel(TO* __restrict__ out, const T* __restrict__ x, int64_t x_ld, int T_rows,
                      int in_dim, SliceTable st, int S, int r_max,
                      const int32_t* __restrict__ token_to_slot, float scaling) {
  const int t = blockIdx.x;
  const int slot = token_to_slot[t];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const bool active = slot >= 0 && slot < S;
  const T* xr = x + (int64_t)t * x_ld;
  for (int q = warp; q < st.n * r_max; q += nwarps) {
    const int s = q / r_max, j = q - s * r_max;
    float acc = 0.f;
    if (active) {
      const T* arow = static_cast<const T*>(st.a[s]) + ((int64_t)slot * r_max + j) * in_dim;
      for (int k = lane; k < in_dim; k += 32) acc += to_float(xr[k]) * to_float(arow[k]);
      acc = warp_sum(acc) * scaling;
    }
    if (lane == 0) out[((int64_t)s * T_rows + t) * r_max + j] = from_float<TO>(acc);
  }
}

// y[t, col_s + o] (+)= tmp[s, t, :] . B_s[slot][o, :]
// (nanovllm_voxcpm/lora_ops/triton_ops/lora_expand_op.py:94-170).
template <typename T, typename TI>
__global__ void __launch_bounds__(kGenericThreads)
generic_expand_kernel(T* __restrict__ y, int64_t y_ld, const TI* __restrict__ tmp, int T_rows,
                      SliceTable st, int S, int r_max,
                      const int32_t* __restrict__ token_to_slot, int add_inputs) {
  extern __shared__ float ts[];  // [n, r_max]
  const int t = blockIdx.x;
  const int slot = token_to_slot[t];
  if (slot < 0 || slot >= S) return;
  for (int q = threadIdx.x; q < st.n * r_max; q += blockDim.x) {
    const int s = q / r_max, j = q - s * r_max;
    ts[q] = to_float(tmp[((int64_t)s * T_rows + t) * r_max + j]);
  }
  __syncthreads();
  for (int s = 0; s < st.n; ++s) {
    const int out = st.out[s];
    if (out == 0) continue;
    const T* b = static_cast<const T*>(st.b[s]) + (int64_t)slot * out * r_max;
    const float* tr = ts + s * r_max;
    T* yr = y + (int64_t)t * y_ld + st.col[s];
    for (int o = threadIdx.x; o < out; o += blockDim.x) {
      const T* brow = b + (int64_t)o * r_max;
      float acc = 0.f;
      for (int j = 0; j < r_max; ++j) acc += tr[j] * to_float(brow[j]);
      yr[o] = from_float<T>(add_inputs ? to_float(yr[o]) + acc : acc);
    }
  }
}

}  // namespace b200lora
