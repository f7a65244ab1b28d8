// Memory-bound glue of a decoder layer around the four projections, one launch each:
//   add_rmsnorm   : hidden = residual + delta; normed = rms_norm(hidden) * weight
//                   (nanovllm_voxcpm/models/voxcpm2/model.py:291-297 with layers/layernorm.py:18-32)
//   rope_kv_store : rotate q and k of the packed qkv rows in place (fp32 math, cos / sin looked up by
//                   position) and copy the rotated k and v rows into the paged cache at slot_mapping
//                   (models/voxcpm2/model.py:81-94, model_utils_rope.py:50-63, layers/attention.py:10-49)
//   silu_mul      : out = silu(gate) * up of the packed gate_up rows (layers/activation.py:11-14)
// The reference runs each of these as a chain of elementwise torch / Inductor / Triton kernels with the
// intermediates in HBM; here every row is read once and written once.
#pragma once

#include "bgmv_fused.cuh"  // aligned16
#include "common.cuh"

namespace b200lora {

constexpr int kGlueThreads = 256;
constexpr int kNormMaxVec = 16;  // 16-byte vectors per lane kept in registers: rows up to 32 * 16 * 8 = 4096 wide

template <typename T>
struct Vec8 {
  uint4 raw;
  __device__ __forceinline__ float get(int i) const { return to_float<T>(reinterpret_cast<const T*>(&raw)[i]); }
  __device__ __forceinline__ void set(int i, float v) { reinterpret_cast<T*>(&raw)[i] = from_float<T>(v); }
};

// One warp per row. `residual` may be null (plain rms_norm of x); `hidden_out` may be null or alias
// `residual` / `x`. norm_of_rounded_sum = 1: the norm sees the sum rounded to T (hidden = residual + x,
// then rms_norm(hidden), the decoder layer's form); 0: it sees the fp32 sum (RMSNorm.add_rms_forward).
template <typename T, int NV>
__global__ void __launch_bounds__(kGlueThreads) add_rmsnorm_kernel(T* __restrict__ normed, int64_t normed_ld,
                                                                   T* hidden_out, int64_t hidden_ld, const T* x,
                                                                   int64_t x_ld, const T* residual, int64_t res_ld,
                                                                   const T* __restrict__ weight, int T_rows, int H,
                                                                   float eps, int norm_of_rounded_sum) {
  // a multi-LoRA launch that follows in the stream may start its weight fetch now (it waits for this
  // kernel's completion before it touches activations)
  griddep_launch_dependents();
  const int row = blockIdx.x * (kGlueThreads / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= T_rows) return;
  const int nvec = H >> 3;  // 8 elements per vector; lane takes vectors lane, lane + 32, ...
  float vals[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      Vec8<T> a, b;
      a.raw = *reinterpret_cast<const uint4*>(x + (int64_t)row * x_ld + 8 * v);
      if (residual != nullptr) b.raw = *reinterpret_cast<const uint4*>(residual + (int64_t)row * res_ld + 8 * v);
      Vec8<T> h;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float s = a.get(j);
        if (residual != nullptr) {
          s = b.get(j) + s;
          h.set(j, s);
          if (norm_of_rounded_sum) s = h.get(j);
        } else {
          h.set(j, s);
        }
        vals[i][j] = s;
        ss += s * s;
      }
      if (hidden_out != nullptr) *reinterpret_cast<uint4*>(hidden_out + (int64_t)row * hidden_ld + 8 * v) = h.raw;
    }
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)H + eps);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      Vec8<T> w, o;
      w.raw = *reinterpret_cast<const uint4*>(weight + 8 * v);
#pragma unroll
      for (int j = 0; j < 8; ++j) o.set(j, vals[i][j] * rstd * w.get(j));
      *reinterpret_cast<uint4*>(normed + (int64_t)row * normed_ld + 8 * v) = o.raw;
    }
  }
}

template <typename T>
inline int add_rmsnorm_launch_t(void* normed, int64_t normed_ld, void* hidden_out, int64_t hidden_ld, const void* x,
                                int64_t x_ld, const void* residual, int64_t res_ld, const void* weight, int T_rows, int H,
                                float eps, int rounded, cudaStream_t stream) {
  const int rows_per_cta = kGlueThreads / 32;
  const dim3 grid((unsigned)((T_rows + rows_per_cta - 1) / rows_per_cta));
  const int nv = (H / 8 + 31) / 32;
#define B200_NORM_CASE(NV)                                                                                              \
  add_rmsnorm_kernel<T, NV><<<grid, kGlueThreads, 0, stream>>>(                                                         \
      static_cast<T*>(normed), normed_ld, static_cast<T*>(hidden_out), hidden_ld, static_cast<const T*>(x), x_ld,       \
      static_cast<const T*>(residual), res_ld, static_cast<const T*>(weight), T_rows, H, eps, rounded)
  if (nv <= 2) B200_NORM_CASE(2);
  else if (nv <= 4) B200_NORM_CASE(4);
  else if (nv <= 8) B200_NORM_CASE(8);
  else B200_NORM_CASE(16);
#undef B200_NORM_CASE
  return check_launch("add_rmsnorm_kernel");
}

inline int add_rmsnorm_launch(void* normed, int64_t normed_ld, void* hidden_out, int64_t hidden_ld, const void* x,
                              int64_t x_ld, const void* residual, int64_t res_ld, const void* weight, int T_rows, int H,
                              float eps, int rounded, int dtype, cudaStream_t stream) {
  if (T_rows < 0 || H <= 0) return fail(B200_LORA_EINVAL, "add_rmsnorm: bad shape T=%d H=%d", T_rows, H);
  if (T_rows == 0) return B200_LORA_OK;
  if (normed == nullptr || x == nullptr || weight == nullptr) return fail(B200_LORA_EINVAL, "add_rmsnorm: null pointer");
  if (dtype != B200_LORA_BF16 && dtype != B200_LORA_F16)
    return fail(B200_LORA_EUNSUPPORTED, "add_rmsnorm: bf16 and fp16 only");
  if (H % 8 != 0 || H > 32 * kNormMaxVec * 8)
    return fail(B200_LORA_EUNSUPPORTED, "add_rmsnorm: width %d (needs a multiple of 8 up to %d)", H, 32 * kNormMaxVec * 8);
  if (!aligned16(normed) || !aligned16(x) || !aligned16(weight) || !aligned16(hidden_out) || !aligned16(residual) ||
      normed_ld % 8 || x_ld % 8 || (hidden_out && hidden_ld % 8) || (residual && res_ld % 8))
    return fail(B200_LORA_EUNSUPPORTED, "add_rmsnorm: rows must start on 16-byte boundaries");
  if (dtype == B200_LORA_BF16)
    return add_rmsnorm_launch_t<__nv_bfloat16>(normed, normed_ld, hidden_out, hidden_ld, x, x_ld, residual, res_ld, weight,
                                               T_rows, H, eps, rounded, stream);
  return add_rmsnorm_launch_t<__half>(normed, normed_ld, hidden_out, hidden_ld, x, x_ld, residual, res_ld, weight, T_rows, H,
                                      eps, rounded, stream);
}

// ------------------------------------------------------------------------------------------ RoPE + KV store
struct RopeKvParams {
  void* qkv; int64_t qkv_ld;          // [T, (Hq + 2 Hk) * D], q | k | v
  int T, Hq, Hk, D;
  const int64_t* positions;           // [T]
  const void* cos; const void* sin;   // [max_pos, table_dim], table_dim = D (the reference's cache) or D / 2
  int table_dim, table_dtype, max_pos;
  void* k_cache; void* v_cache;       // [slots, Hk * D], may be null (no cache: rotation only)
  const int32_t* slot_mapping;        // [T], -1 = do not store
  int apply_rope;
};

__device__ __forceinline__ float table_at(const void* tab, int dtype, int64_t idx) {
  if (dtype == B200_LORA_F32) return static_cast<const float*>(tab)[idx];
  if (dtype == B200_LORA_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(tab)[idx]);
  return __half2float(static_cast<const __half*>(tab)[idx]);
}

__device__ __forceinline__ void table_load8(const void* tab, int dtype, int64_t idx, float (&out)[8]) {
  if (dtype == B200_LORA_F32) {
    const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(tab) + idx);
    const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(tab) + idx + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  } else if (dtype == B200_LORA_BF16) {
    Vec8<__nv_bfloat16> v;
    v.raw = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(tab) + idx);
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = v.get(e);
  } else {
    Vec8<__half> v;
    v.raw = *reinterpret_cast<const uint4*>(static_cast<const __half*>(tab) + idx);
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = v.get(e);
  }
}

// Work items of 16 bytes, flat over (token, item): a rotation item is (head, 8 adjacent columns j..j+7 of the
// first half) -> y[j] = x[j] * cos[j] - x[j + D/2] * sin[j], y[j + D/2] = x[j + D/2] * cos[j + D/2] + x[j] * sin[j + D/2],
// each product and the sum rounded separately in fp32 as the reference's elementwise chain does; a rotated k
// vector also goes to the cache. The remaining items of a token copy its v row (and its k row when nothing is
// rotated) to the cache.
constexpr int kRopeThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kRopeThreads) rope_kv_store_kernel(const RopeKvParams p) {
  griddep_launch_dependents();
  const int half = p.D >> 1, vec_per_half = half >> 3;
  const int q_size = p.Hq * p.D, kv_size = p.Hk * p.D, kv_vecs = kv_size >> 3;
  const int rot_items = p.apply_rope ? (p.Hq + p.Hk) * vec_per_half : 0;
  const bool store = p.k_cache != nullptr && p.slot_mapping != nullptr;
  const int copy_items = store ? (p.apply_rope ? kv_vecs : 2 * kv_vecs) : 0;
  const int per_tok = rot_items + copy_items;
  const int64_t total = (int64_t)p.T * per_tok;
  const int hi_off = p.table_dim == p.D ? half : 0;
  for (int64_t idx = (int64_t)blockIdx.x * kRopeThreads + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * kRopeThreads) {
    const int tok = (int)(idx / per_tok), it = (int)(idx - (int64_t)tok * per_tok);
    T* row = static_cast<T*>(p.qkv) + (int64_t)tok * p.qkv_ld;
    const int64_t slot = store ? (int64_t)p.slot_mapping[tok] : -1;
    if (it < rot_items) {
      const int head = it / vec_per_half, j = (it - head * vec_per_half) * 8;
      T* h = row + head * p.D;  // k heads follow the q heads directly
      int64_t pos = p.positions[tok];
      pos = pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
      const int64_t tb = pos * p.table_dim + j;
      Vec8<T> lo, hi, olo, ohi;
      lo.raw = *reinterpret_cast<const uint4*>(h + j);
      hi.raw = *reinterpret_cast<const uint4*>(h + half + j);
      // 8 consecutive table entries per operand, fetched as 16-byte vectors (tb is a multiple of 8 entries)
      float c1[8], s1[8], c2[8], s2[8];
      table_load8(p.cos, p.table_dtype, tb, c1);
      table_load8(p.sin, p.table_dtype, tb, s1);
      if (hi_off) {
        table_load8(p.cos, p.table_dtype, tb + hi_off, c2);
        table_load8(p.sin, p.table_dtype, tb + hi_off, s2);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float x1 = lo.get(e), x2 = hi.get(e);
        const float cc2 = hi_off ? c2[e] : c1[e], ss2 = hi_off ? s2[e] : s1[e];
        olo.set(e, __fadd_rn(__fmul_rn(x1, c1[e]), __fmul_rn(-x2, s1[e])));
        ohi.set(e, __fadd_rn(__fmul_rn(x2, cc2), __fmul_rn(x1, ss2)));
      }
      *reinterpret_cast<uint4*>(h + j) = olo.raw;
      *reinterpret_cast<uint4*>(h + half + j) = ohi.raw;
      if (slot >= 0 && head >= p.Hq) {
        T* d = static_cast<T*>(p.k_cache) + slot * kv_size + (head - p.Hq) * p.D;
        *reinterpret_cast<uint4*>(d + j) = olo.raw;
        *reinterpret_cast<uint4*>(d + half + j) = ohi.raw;
      }
    } else if (slot >= 0) {
      int c = it - rot_items;  // v vectors first, then (no rotation) the k vectors
      const bool is_v = c < kv_vecs;
      if (!is_v) c -= kv_vecs;
      const T* src = row + q_size + (is_v ? kv_size : 0) + 8 * c;
      T* dst = static_cast<T*>(is_v ? p.v_cache : p.k_cache) + slot * kv_size + 8 * c;
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
    }
  }
}

inline int rope_kv_store_launch(const RopeKvParams& p, int dtype, cudaStream_t stream) {
  if (p.T < 0 || p.Hq < 0 || p.Hk < 0 || p.D <= 0) return fail(B200_LORA_EINVAL, "rope_kv_store: bad shape");
  if (p.T == 0) return B200_LORA_OK;
  if (p.qkv == nullptr) return fail(B200_LORA_EINVAL, "rope_kv_store: null qkv");
  if (dtype != B200_LORA_BF16 && dtype != B200_LORA_F16)
    return fail(B200_LORA_EUNSUPPORTED, "rope_kv_store: bf16 and fp16 only");
  if (p.D % 16 != 0 || p.qkv_ld % 8 != 0 || !aligned16(p.qkv) || !aligned16(p.k_cache) || !aligned16(p.v_cache) ||
      !aligned16(p.cos) || !aligned16(p.sin))
    return fail(B200_LORA_EUNSUPPORTED, "rope_kv_store: head_dim must be a multiple of 16 and the row pitch of 8 elements, "
                                        "rows and tables 16-byte aligned");
  if ((p.k_cache == nullptr) != (p.v_cache == nullptr)) return fail(B200_LORA_EINVAL, "rope_kv_store: one cache is null");
  if (p.apply_rope) {
    if (p.positions == nullptr || p.cos == nullptr || p.sin == nullptr || p.max_pos <= 0)
      return fail(B200_LORA_EINVAL, "rope_kv_store: rotation needs positions and cos / sin tables");
    if (p.table_dim != p.D && p.table_dim != p.D / 2)
      return fail(B200_LORA_EINVAL, "rope_kv_store: table width %d is neither head_dim nor head_dim / 2", p.table_dim);
    if (p.table_dtype != B200_LORA_F32 && p.table_dtype != B200_LORA_BF16 && p.table_dtype != B200_LORA_F16)
      return fail(B200_LORA_EINVAL, "rope_kv_store: bad table dtype");
  }
  const bool store = p.k_cache != nullptr && p.slot_mapping != nullptr;
  const int per_tok = (p.apply_rope ? (p.Hq + p.Hk) * (p.D / 16) : 0) + (store ? (p.apply_rope ? 1 : 2) * p.Hk * p.D / 8 : 0);
  if (per_tok == 0) return B200_LORA_OK;
  const int64_t want = ((int64_t)p.T * per_tok + kRopeThreads - 1) / kRopeThreads;
  const unsigned grid = (unsigned)std::min<int64_t>(want, 148 * 16);
  if (dtype == B200_LORA_BF16) rope_kv_store_kernel<__nv_bfloat16><<<grid, kRopeThreads, 0, stream>>>(p);
  else rope_kv_store_kernel<__half><<<grid, kRopeThreads, 0, stream>>>(p);
  return check_launch("rope_kv_store_kernel");
}

// ------------------------------------------------------------------------------------------ SiLU * up
// x [T, 2 * I] (gate | up), out [T, I]; 8 columns per thread, grid-stride over (row, vector).
template <typename T>
__global__ void __launch_bounds__(kGlueThreads) silu_mul_kernel(T* __restrict__ out, int64_t out_ld,
                                                                const T* __restrict__ x, int64_t x_ld, int T_rows, int I) {
  griddep_launch_dependents();
  const int nvec = I >> 3;
  const int64_t total = (int64_t)T_rows * nvec;
  for (int64_t i = (int64_t)blockIdx.x * kGlueThreads + threadIdx.x; i < total; i += (int64_t)gridDim.x * kGlueThreads) {
    const int row = (int)(i / nvec), v = (int)(i - (int64_t)row * nvec);
    Vec8<T> g, u, o;
    g.raw = *reinterpret_cast<const uint4*>(x + (int64_t)row * x_ld + 8 * v);
    u.raw = *reinterpret_cast<const uint4*>(x + (int64_t)row * x_ld + I + 8 * v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = g.get(j);
      o.set(j, a / (1.f + expf(-a)) * u.get(j));
    }
    *reinterpret_cast<uint4*>(out + (int64_t)row * out_ld + 8 * v) = o.raw;
  }
}

inline int silu_mul_launch(void* out, int64_t out_ld, const void* x, int64_t x_ld, int T_rows, int I, int dtype,
                           cudaStream_t stream) {
  if (T_rows < 0 || I <= 0) return fail(B200_LORA_EINVAL, "silu_mul: bad shape");
  if (T_rows == 0) return B200_LORA_OK;
  if (out == nullptr || x == nullptr) return fail(B200_LORA_EINVAL, "silu_mul: null pointer");
  if (dtype != B200_LORA_BF16 && dtype != B200_LORA_F16) return fail(B200_LORA_EUNSUPPORTED, "silu_mul: bf16 and fp16 only");
  if (I % 8 != 0 || out_ld % 8 != 0 || x_ld % 8 != 0 || !aligned16(out) || !aligned16(x))
    return fail(B200_LORA_EUNSUPPORTED, "silu_mul: widths and pitches must be multiples of 8 elements, rows 16-byte aligned");
  const int64_t total = (int64_t)T_rows * (I / 8);
  const int64_t want = (total + kGlueThreads - 1) / kGlueThreads;
  const unsigned grid = (unsigned)std::min<int64_t>(want, 148 * 16);  // a multiple of the SM count when the batch is large
  if (dtype == B200_LORA_BF16)
    silu_mul_kernel<__nv_bfloat16><<<grid, kGlueThreads, 0, stream>>>(static_cast<__nv_bfloat16*>(out), out_ld,
                                                                     static_cast<const __nv_bfloat16*>(x), x_ld, T_rows, I);
  else
    silu_mul_kernel<__half><<<grid, kGlueThreads, 0, stream>>>(static_cast<__half*>(out), out_ld,
                                                               static_cast<const __half*>(x), x_ld, T_rows, I);
  return check_launch("silu_mul_kernel");
}

}  // namespace b200lora
