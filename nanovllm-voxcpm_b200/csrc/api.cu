// C ABI of the B200 multi-LoRA library: argument checks + kernel dispatch.
// Declarations and the reference interface each entry point replaces: include/b200_lora.h
#include "common.cuh"
#include "generic.cuh"
#include "bgmv_fused.cuh"
#include "metadata.cuh"
#include "tp_exchange.cuh"
#include "slot_loader.cuh"
#include "glue.cuh"
#include "sgmv_tc.cuh"
#include "gemm_tc.cuh"

using namespace b200lora;

namespace {

int fill_slices(SliceTable& st, int n_slices, const void* const* a_slabs,
                const void* const* b_slabs, const int32_t* out_sizes,
                const int32_t* col_offsets, bool need_a, bool need_b) {
  if (n_slices < 1 || n_slices > B200_LORA_MAX_SLICES)
    return fail(B200_LORA_EINVAL, "n_slices=%d outside [1,%d]", n_slices, B200_LORA_MAX_SLICES);
  st.n = n_slices;
  for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) {
    st.a[s] = st.b[s] = nullptr;
    st.out[s] = st.col[s] = 0;
  }
  for (int s = 0; s < n_slices; ++s) {
    st.out[s] = out_sizes ? out_sizes[s] : 1;
    st.col[s] = col_offsets ? col_offsets[s] : 0;
    if (st.out[s] < 0 || st.col[s] < 0)
      return fail(B200_LORA_EINVAL, "slice %d: negative width/offset", s);
    if (need_a) {
      st.a[s] = a_slabs ? a_slabs[s] : nullptr;
      if (st.a[s] == nullptr && st.out[s] > 0) return fail(B200_LORA_EINVAL, "slice %d: null lora_A slab", s);
    }
    if (need_b) {
      st.b[s] = b_slabs ? b_slabs[s] : nullptr;
      if (st.b[s] == nullptr && st.out[s] > 0) return fail(B200_LORA_EINVAL, "slice %d: null lora_B slab", s);
    }
  }
  return B200_LORA_OK;
}

// y[row, slice columns] = -0.0 (sign bit only) for every slice; elem = bytes per element
__global__ void fill_neg_zero_kernel(void* y, int64_t y_ld, const SliceTable st, int elem) {
  const int64_t row = blockIdx.x;
  for (int s = 0; s < st.n; ++s) {
    if (elem == 2) {
      uint16_t* dst = static_cast<uint16_t*>(y) + row * y_ld + st.col[s];
      for (int i = threadIdx.x; i < st.out[s]; i += blockDim.x) dst[i] = 0x8000u;
    } else {
      uint32_t* dst = static_cast<uint32_t*>(y) + row * y_ld + st.col[s];
      for (int i = threadIdx.x; i < st.out[s]; i += blockDim.x) dst[i] = 0x80000000u;
    }
  }
}

bool valid_dtype(int d) { return d == B200_LORA_BF16 || d == B200_LORA_F16 || d == B200_LORA_F32; }

template <typename T>
int launch_generic_add(void* y, int64_t y_ld, const void* x, int64_t x_ld, int T_rows, int in_dim,
                       const SliceTable& st, int S, int r_max, const int32_t* rank_per_slot,
                       const float* scale_per_slot, const int32_t* token_to_slot, float scaling,
                       cudaStream_t stream) {
  const size_t smem = sizeof(float) * st.n * r_max;
  generic_add_kernel<T><<<T_rows, kGenericThreads, smem, stream>>>(
      static_cast<T*>(y), y_ld, static_cast<const T*>(x), x_ld, in_dim, st, S, r_max,
      rank_per_slot, scale_per_slot, token_to_slot, scaling);
  return check_launch("generic_add_kernel");
}

template <typename T, typename TO>
int launch_generic_shrink(void* out, const void* x, int64_t x_ld, int T_rows, int in_dim,
                          const SliceTable& st, int S, int r_max, const int32_t* token_to_slot,
                          float scaling, cudaStream_t stream) {
  generic_shrink_kernel<T, TO><<<T_rows, kGenericThreads, 0, stream>>>(
      static_cast<TO*>(out), static_cast<const T*>(x), x_ld, T_rows, in_dim, st, S, r_max,
      token_to_slot, scaling);
  return check_launch("generic_shrink_kernel");
}

template <typename T, typename TI>
int launch_generic_expand(void* y, int64_t y_ld, const void* tmp, int T_rows, const SliceTable& st,
                          int S, int r_max, const int32_t* token_to_slot, int add_inputs,
                          cudaStream_t stream) {
  const size_t smem = sizeof(float) * st.n * r_max;
  generic_expand_kernel<T, TI><<<T_rows, kGenericThreads, smem, stream>>>(
      static_cast<T*>(y), y_ld, static_cast<const TI*>(tmp), T_rows, st, S, r_max, token_to_slot,
      add_inputs);
  return check_launch("generic_expand_kernel");
}

}  // namespace

extern "C" {

int lora_b200_version(void) { return B200_LORA_ABI_VERSION; }

const char* lora_b200_last_error(void) { return error_buffer(); }

int lora_b200_set_option(int32_t key, int32_t value) {
  if (key == B200_LORA_OPT_CLUSTER) {
    if (value != 0 && value != 1 && value != 2 && value != 4 && value != 8)
      return fail(B200_LORA_EINVAL, "cluster size %d not in {0,1,2,4,8}", value);
    bgmv_options().cluster = value;
    return B200_LORA_OK;
  }
  if (key == B200_LORA_OPT_PDL) {
    bgmv_options().pdl = value != 0;
    return B200_LORA_OK;
  }
  if (key == B200_LORA_OPT_RING_KB) {
    if (value < 0 || value > 227) return fail(B200_LORA_EINVAL, "ring size %d KB outside [0, 227]", value);
    bgmv_options().ring_kb = value;
    return B200_LORA_OK;
  }
  if (key == B200_LORA_OPT_PEER_POLL_LIMIT) {
    if (value < 0) return fail(B200_LORA_EINVAL, "poll limit %d is negative", value);
    tp_spin_limit() = value == 0 ? kTpSpinLimit : value;
    return B200_LORA_OK;
  }
  if (key == B200_LORA_OPT_KSPLIT) {
    bgmv_options().ksplit = value != 0;
    return B200_LORA_OK;
  }
  return fail(B200_LORA_EINVAL, "unknown option %d", key);
}

int lora_b200_build_metadata(const int32_t* token_to_slot, int32_t T, int32_t S, int32_t convention,
                             int32_t* sorted_idx, int32_t* slot_ids, int32_t* counts, int32_t* offsets,
                             int32_t* info, void* stream) {
  return build_metadata(token_to_slot, T, S, convention, sorted_idx, slot_ids, counts, offsets, info,
                        static_cast<cudaStream_t>(stream));
}

int lora_b200_load_slot(const void* staging, int32_t n_desc, int64_t max_elems, void* stream) {
  return slot_load_launch(staging, n_desc, max_elems, static_cast<cudaStream_t>(stream));
}

int lora_b200_glue_add_rmsnorm(void* normed, int64_t normed_ld, void* hidden_out, int64_t hidden_ld, const void* x,
                               int64_t x_ld, const void* residual, int64_t residual_ld, const void* weight, int32_t T,
                               int32_t hidden, float eps, int32_t norm_of_rounded_sum, int32_t dtype, void* stream) {
  return add_rmsnorm_launch(normed, normed_ld, hidden_out, hidden_ld, x, x_ld, residual, residual_ld, weight, T, hidden, eps,
                            norm_of_rounded_sum, dtype, static_cast<cudaStream_t>(stream));
}

int lora_b200_glue_rope_kv_store(void* qkv, int64_t qkv_ld, int32_t T, int32_t num_heads, int32_t num_kv_heads,
                                 int32_t head_dim, const int64_t* positions, const void* cos_table, const void* sin_table,
                                 int32_t table_dim, int32_t table_dtype, int32_t max_position, void* k_cache, void* v_cache,
                                 const int32_t* slot_mapping, int32_t dtype, void* stream) {
  RopeKvParams p;
  p.qkv = qkv; p.qkv_ld = qkv_ld; p.T = T; p.Hq = num_heads; p.Hk = num_kv_heads; p.D = head_dim;
  p.positions = positions; p.cos = cos_table; p.sin = sin_table;
  p.table_dim = table_dim; p.table_dtype = table_dtype; p.max_pos = max_position;
  p.k_cache = k_cache; p.v_cache = v_cache; p.slot_mapping = slot_mapping;
  p.apply_rope = (cos_table != nullptr || sin_table != nullptr || positions != nullptr) ? 1 : 0;
  return rope_kv_store_launch(p, dtype, static_cast<cudaStream_t>(stream));
}

int lora_b200_glue_silu_mul(void* out, int64_t out_ld, const void* gate_up, int64_t gate_up_ld, int32_t T,
                            int32_t intermediate, int32_t dtype, void* stream) {
  return silu_mul_launch(out, out_ld, gate_up, gate_up_ld, T, intermediate, dtype, static_cast<cudaStream_t>(stream));
}

size_t lora_b200_tp_exchange_bytes(int32_t tp, int32_t capacity) { return tp_exchange_bytes(tp, capacity); }

int lora_b200_tp_allreduce(const float* partial, float* out, int32_t count, void* const* peer_buffers, int32_t rank,
                           int32_t tp, int32_t capacity, void* stream) {
  return tp_allreduce_launch(partial, out, count, peer_buffers, rank, tp, capacity, static_cast<cudaStream_t>(stream));
}

#ifdef B200_TRACE
// Tuning builds only: copies the phase timeline of the last fused-decode launch.
int lora_b200_debug_trace(long long* out, int32_t n_values) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_b200_trace, sizeof(long long) * (size_t)n_values);
  return e == cudaSuccess ? 0 : B200_LORA_ECUDA;
}
#endif

int lora_b200_device_status(int32_t* status, int32_t reset) {
  if (status == nullptr) return fail(B200_LORA_EINVAL, "null status pointer");
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_b200_status, sizeof(int));
  if (e != cudaSuccess) return fail(B200_LORA_ECUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
  *status = v;
  if (reset) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_b200_status, &zero, sizeof(int));
    if (e != cudaSuccess) return fail(B200_LORA_ECUDA, "cudaMemcpyToSymbol: %s", cudaGetErrorString(e));
  }
  return B200_LORA_OK;
}

int lora_b200_linear_lora(void* y, int64_t y_ld, const void* x, int64_t x_ld, int32_t T, int32_t in_dim,
                          const void* weight, int64_t w_ld, int32_t out_total, const void* bias, int32_t n_slices,
                          const void* const* a_slabs, const void* const* b_slabs, const int32_t* out_sizes,
                          const int32_t* col_offsets, int32_t S, int32_t r_max, const float* scale_per_slot,
                          const int32_t* token_to_slot, float scaling, void* workspace, size_t workspace_bytes,
                          void* stream) {
  if (T < 0 || in_dim < 1 || out_total < 1) return fail(B200_LORA_EINVAL, "bad sizes T=%d in=%d out=%d", T, in_dim, out_total);
  if (T == 0) return B200_LORA_OK;
  if (y == nullptr || x == nullptr || weight == nullptr) return fail(B200_LORA_EINVAL, "null y / x / weight");
  if (y_ld < out_total || x_ld < in_dim || w_ld < in_dim) return fail(B200_LORA_EINVAL, "row stride smaller than row");
  LinearProblem lp;
  lp.weight = weight; lp.w_ld = w_ld; lp.n_total = out_total; lp.bias = bias;
  SliceTable st;
  st.n = 0;
  for (int s = 0; s < B200_LORA_MAX_SLICES; ++s) { st.a[s] = st.b[s] = nullptr; st.out[s] = st.col[s] = 0; }
  if (n_slices > 0 && token_to_slot != nullptr) {
    if (S < 1 || r_max < 1) return fail(B200_LORA_EINVAL, "bad sizes S=%d r_max=%d", S, r_max);
    if (out_sizes == nullptr || col_offsets == nullptr) return fail(B200_LORA_EINVAL, "null out_sizes / col_offsets");
    if (int rc = fill_slices(st, n_slices, a_slabs, b_slabs, out_sizes, col_offsets, true, true)) return rc;
    for (int s = 0; s < st.n; ++s)
      if (st.col[s] + st.out[s] > out_total) return fail(B200_LORA_EINVAL, "slice %d exceeds the output width", s);
  }
  lp.lora.y = y; lp.lora.y_ld = y_ld; lp.lora.x = x; lp.lora.x_ld = x_ld; lp.lora.T = T; lp.lora.in_dim = in_dim;
  lp.lora.S = S; lp.lora.r_max = r_max; lp.lora.st = st; lp.lora.scale_per_slot = scale_per_slot;
  lp.lora.token_to_slot = token_to_slot; lp.lora.scaling = scaling;
  return linear_lora_launch(lp, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

size_t lora_b200_workspace_bytes(int32_t T, int32_t n_slices, int32_t r_max) {
  if (T < 0 || n_slices < 1 || r_max < 1) return 0;
  return sgmv_workspace_bytes(T, n_slices, r_max);
}

int lora_b200_shrink_allreduce_expand(void* y, int64_t y_ld, const void* x, int64_t x_ld, int32_t T, int32_t in_dim,
                                      int32_t n_slices, const void* const* a_slabs, const void* const* b_slabs,
                                      const int32_t* out_sizes, const int32_t* col_offsets, int32_t S, int32_t r_max,
                                      const int32_t* rank_per_slot, const float* scale_per_slot,
                                      const int32_t* token_to_slot, const int32_t* sorted_idx, const int32_t* slot_ids,
                                      const int32_t* counts, const int32_t* offsets, int32_t n_buckets, float scaling,
                                      int32_t dtype, float* tmp, void* const* peer_buffers, int32_t rank, int32_t tp,
                                      int32_t capacity, void* stream) {
  if (!valid_dtype(dtype)) return fail(B200_LORA_EINVAL, "unknown dtype %d", dtype);
  if (T < 0 || in_dim < 1 || S < 1 || r_max < 1)
    return fail(B200_LORA_EINVAL, "bad sizes T=%d in=%d S=%d r_max=%d", T, in_dim, S, r_max);
  if (T == 0) return B200_LORA_OK;
  if (y == nullptr || x == nullptr || token_to_slot == nullptr || tmp == nullptr)
    return fail(B200_LORA_EINVAL, "null y / x / token_to_slot / tmp");
  if (out_sizes == nullptr || col_offsets == nullptr) return fail(B200_LORA_EINVAL, "null out_sizes / col_offsets");
  if (tp < 1 || rank < 0 || rank >= tp) return fail(B200_LORA_EINVAL, "rank %d of %d", rank, tp);
  if (tp > 1 && peer_buffers == nullptr) return fail(B200_LORA_EINVAL, "null peer_buffers with tp=%d", tp);
  SliceTable st;
  if (int rc = fill_slices(st, n_slices, a_slabs, b_slabs, out_sizes, col_offsets, true, true)) return rc;
  int n_act = 0;
  int64_t width = 0;
  for (int s = 0; s < st.n; ++s) {
    if (st.out[s] == 0) return fail(B200_LORA_EUNSUPPORTED, "tensor-parallel exchange: zero-width slice %d", s);
    width = width > (int64_t)st.col[s] + st.out[s] ? width : (int64_t)st.col[s] + st.out[s];
    ++n_act;
  }
  if (y_ld < width || x_ld < in_dim)
    return fail(B200_LORA_EINVAL, "row stride smaller than row: y_ld=%lld (need %lld) x_ld=%lld (need %d)",
                (long long)y_ld, (long long)width, (long long)x_ld, in_dim);
  const int64_t count64 = (int64_t)n_act * T * r_max;
  if (count64 > (int64_t)INT32_MAX || (count64 & 3)) return fail(B200_LORA_EINVAL, "n_slices * T * r_max must be a multiple of 4 below 2^31");
  const int count = (int)count64;
  cudaStream_t st_ = static_cast<cudaStream_t>(stream);
  const bool have_buckets = sorted_idx && slot_ids && counts && offsets && n_buckets > 0;

  BgmvProblem bp;
  bp.y = y; bp.y_ld = y_ld; bp.x = x; bp.x_ld = x_ld; bp.T = T; bp.in_dim = in_dim; bp.st = st;
  bp.S = S; bp.r_max = r_max; bp.rank_per_slot = rank_per_slot; bp.scale_per_slot = scale_per_slot;
  bp.sorted_idx = sorted_idx; bp.slot_ids = slot_ids; bp.counts = counts; bp.offsets = offsets;
  bp.n_buckets = n_buckets; bp.scaling = scaling; bp.tmp_io = tmp;
  BgmvProblem shrink_p = bp, expand_p = bp;
  shrink_p.mode = 1;
  expand_p.mode = 2; expand_p.scaling = 1.0f; expand_p.scale_per_slot = nullptr;  // the scale is already in tmp
  const bool fused_kernels = dtype == B200_LORA_BF16 && have_buckets && bgmv_supported(shrink_p, nullptr) &&
                             bgmv_supported(expand_p, nullptr);
  if (fused_kernels) {
    if (int rc = bgmv_launch(shrink_p, st_)) return rc;
  } else {
    // any dtype / shape: one CTA per token; rows without adapter are zero-filled (they are exchanged too)
    if (r_max > 2048) return fail(B200_LORA_EUNSUPPORTED, "generic kernel: r_max=%d > 2048", r_max);
    if (scale_per_slot != nullptr) return fail(B200_LORA_EUNSUPPORTED, "per-slot scales need the bf16 bucket kernels here");
    int rc;
    if (dtype == B200_LORA_BF16)
      rc = launch_generic_shrink<__nv_bfloat16, float>(tmp, x, x_ld, T, in_dim, st, S, r_max, token_to_slot, scaling, st_);
    else if (dtype == B200_LORA_F16)
      rc = launch_generic_shrink<__half, float>(tmp, x, x_ld, T, in_dim, st, S, r_max, token_to_slot, scaling, st_);
    else
      rc = launch_generic_shrink<float, float>(tmp, x, x_ld, T, in_dim, st, S, r_max, token_to_slot, scaling, st_);
    if (rc) return rc;
  }
  if (tp > 1)
    if (int rc = tp_allreduce_launch(tmp, tmp, count, peer_buffers, rank, tp, capacity, st_)) return rc;
  if (fused_kernels) return bgmv_launch(expand_p, st_);
  if (dtype == B200_LORA_BF16) return launch_generic_expand<__nv_bfloat16, float>(y, y_ld, tmp, T, st, S, r_max, token_to_slot, 1, st_);
  if (dtype == B200_LORA_F16) return launch_generic_expand<__half, float>(y, y_ld, tmp, T, st, S, r_max, token_to_slot, 1, st_);
  return launch_generic_expand<float, float>(y, y_ld, tmp, T, st, S, r_max, token_to_slot, 1, st_);
}

// overwrite = 0: y += delta (lora_b200_add); 1: y = delta, -0.0 in rows without one (lora_b200_delta)
static int add_or_delta(void* y, int64_t y_ld, const void* x, int64_t x_ld, int32_t T, int32_t in_dim,
                        int32_t n_slices, const void* const* a_slabs, const void* const* b_slabs,
                        const int32_t* out_sizes, const int32_t* col_offsets, int32_t S, int32_t r_max,
                        const int32_t* rank_per_slot, const float* scale_per_slot,
                        const int32_t* token_to_slot, const int32_t* sorted_idx, const int32_t* slot_ids,
                        const int32_t* counts, const int32_t* offsets, int32_t n_buckets, float scaling,
                        int32_t dtype, int32_t impl, void* workspace, size_t workspace_bytes,
                        void* stream, int overwrite) {
  if (!valid_dtype(dtype)) return fail(B200_LORA_EINVAL, "unknown dtype %d", dtype);
  if (T < 0 || in_dim < 1 || S < 1 || r_max < 1)
    return fail(B200_LORA_EINVAL, "bad sizes T=%d in=%d S=%d r_max=%d", T, in_dim, S, r_max);
  if (T == 0) return B200_LORA_OK;
  if (y == nullptr || x == nullptr || token_to_slot == nullptr)
    return fail(B200_LORA_EINVAL, "null y / x / token_to_slot");
  if (out_sizes == nullptr || col_offsets == nullptr)
    return fail(B200_LORA_EINVAL, "null out_sizes / col_offsets");
  SliceTable st;
  if (int rc = fill_slices(st, n_slices, a_slabs, b_slabs, out_sizes, col_offsets, true, true)) return rc;
  int64_t width = 0;
  bool any = false;
  for (int s = 0; s < st.n; ++s) {
    width = width > (int64_t)st.col[s] + st.out[s] ? width : (int64_t)st.col[s] + st.out[s];
    any = any || st.out[s] > 0;
  }
  if (!any) return B200_LORA_OK;
  if (y_ld < width || x_ld < in_dim)
    return fail(B200_LORA_EINVAL, "row stride smaller than row: y_ld=%lld (need %lld) x_ld=%lld (need %d)",
                (long long)y_ld, (long long)width, (long long)x_ld, in_dim);
  cudaStream_t st_ = static_cast<cudaStream_t>(stream);
  const bool have_buckets = sorted_idx && slot_ids && counts && offsets && n_buckets > 0;

  BgmvProblem bp;
  bp.y = y; bp.y_ld = y_ld; bp.x = x; bp.x_ld = x_ld; bp.T = T; bp.in_dim = in_dim; bp.st = st;
  bp.S = S; bp.r_max = r_max; bp.rank_per_slot = rank_per_slot; bp.scale_per_slot = scale_per_slot;
  bp.sorted_idx = sorted_idx; bp.slot_ids = slot_ids; bp.counts = counts; bp.offsets = offsets;
  bp.n_buckets = n_buckets; bp.scaling = scaling;

  SgmvProblem sp;
  sp.y = y; sp.y_ld = y_ld; sp.x = x; sp.x_ld = x_ld; sp.T = T; sp.in_dim = in_dim; sp.S = S; sp.r_max = r_max;
  sp.st = st; sp.scale_per_slot = scale_per_slot; sp.token_to_slot = token_to_slot; sp.scaling = scaling;

  if (overwrite) {
    // decode batches: the row-split kernel writes the delta (and the -0.0 rows) itself; everything else
    // fills y with -0.0 first and then adds as usual (-0.0 + d == d)
    bp.mode = 3;
    bp.token_to_slot = token_to_slot;
    const bool decode_like = T < kSgmvAutoMinTokens || T < 32 * n_buckets;
    if (dtype == B200_LORA_BF16 && have_buckets &&
        (impl == B200_LORA_IMPL_BGMV || (impl == B200_LORA_IMPL_AUTO && decode_like)) && bgmv_supported(bp, nullptr))
      return bgmv_launch(bp, st_);
    bp.mode = 0;
    bp.token_to_slot = nullptr;
    // prefill batches: the tile kernel stores the delta tiles instead of reduce-adding them
    {
      int n_act = 0;
      for (int s = 0; s < st.n; ++s) n_act += st.out[s] > 0;
      if (dtype == B200_LORA_BF16 && (impl == B200_LORA_IMPL_SGMV || (impl == B200_LORA_IMPL_AUTO && !decode_like)) &&
          sgmv_supported(sp, nullptr) && prefill_overwrite_ok(st) && workspace != nullptr &&
          workspace_bytes >= sgmv_workspace_bytes(T, n_act, r_max))
        return prefill_add_launch(sp, workspace, workspace_bytes, st_, true);
    }
    fill_neg_zero_kernel<<<(unsigned)T, 128, 0, st_>>>(y, y_ld, st, dtype == B200_LORA_F32 ? 4 : 2);
    if (int rc = check_launch("fill_neg_zero_kernel")) return rc;
  }

  if (impl == B200_LORA_IMPL_AUTO) {
    // Long batches (prefill) go to the tensor-core kernels when scratch memory was supplied, decode
    // batches to the fused kernel, everything else (other dtypes, odd shapes) to the generic one.
    int n_act = 0;
    for (int s = 0; s < st.n; ++s) n_act += st.out[s] > 0;
    const bool bgmv_ok = dtype == B200_LORA_BF16 && have_buckets && bgmv_supported(bp, nullptr);
    // The prefill kernels tile rows in token order and pay one stage per run of equal slot, so they
    // want request-contiguous rows: with bucket arrays at hand, fewer than 32 rows per bucket on
    // average means a decode-like batch (slots scattered over the rows) and goes to the bucket kernel.
    const bool scattered = bgmv_ok && T < 32 * n_buckets;
    if (dtype == B200_LORA_BF16 && T >= kSgmvAutoMinTokens && !scattered && sgmv_supported(sp, nullptr) &&
        workspace != nullptr && workspace_bytes >= sgmv_workspace_bytes(T, n_act, r_max))
      impl = B200_LORA_IMPL_SGMV;
    else if (bgmv_ok)
      impl = B200_LORA_IMPL_BGMV;
    else
      impl = B200_LORA_IMPL_GENERIC;
  }
  switch (impl) {
    case B200_LORA_IMPL_GENERIC:
      if (r_max > 2048) return fail(B200_LORA_EUNSUPPORTED, "generic kernel: r_max=%d > 2048", r_max);
      if (dtype == B200_LORA_BF16)
        return launch_generic_add<__nv_bfloat16>(y, y_ld, x, x_ld, T, in_dim, st, S, r_max, rank_per_slot,
                                                 scale_per_slot, token_to_slot, scaling, st_);
      if (dtype == B200_LORA_F16)
        return launch_generic_add<__half>(y, y_ld, x, x_ld, T, in_dim, st, S, r_max, rank_per_slot,
                                          scale_per_slot, token_to_slot, scaling, st_);
      return launch_generic_add<float>(y, y_ld, x, x_ld, T, in_dim, st, S, r_max, rank_per_slot,
                                       scale_per_slot, token_to_slot, scaling, st_);
    case B200_LORA_IMPL_BGMV: {
      if (dtype != B200_LORA_BF16) return fail(B200_LORA_EUNSUPPORTED, "fused decode kernel is bf16 only");
      if (!have_buckets) return fail(B200_LORA_EINVAL, "fused decode kernel needs the bucket arrays");
      const char* why = nullptr;
      if (bgmv_supported(bp, &why)) return bgmv_launch(bp, st_);
      return fail(B200_LORA_EUNSUPPORTED, "fused decode kernel: %s", why);
    }
    case B200_LORA_IMPL_SGMV:
      if (dtype != B200_LORA_BF16) return fail(B200_LORA_EUNSUPPORTED, "prefill kernels are bf16 only");
      return prefill_add_launch(sp, workspace, workspace_bytes, st_);
    default:
      return fail(B200_LORA_EUNSUPPORTED, "impl %d is not available", impl);
  }
}

int lora_b200_add(void* y, int64_t y_ld, const void* x, int64_t x_ld, int32_t T, int32_t in_dim,
                  int32_t n_slices, const void* const* a_slabs, const void* const* b_slabs,
                  const int32_t* out_sizes, const int32_t* col_offsets, int32_t S, int32_t r_max,
                  const int32_t* rank_per_slot, const float* scale_per_slot,
                  const int32_t* token_to_slot, const int32_t* sorted_idx, const int32_t* slot_ids,
                  const int32_t* counts, const int32_t* offsets, int32_t n_buckets, float scaling,
                  int32_t dtype, int32_t impl, void* workspace, size_t workspace_bytes,
                  void* stream) {
  return add_or_delta(y, y_ld, x, x_ld, T, in_dim, n_slices, a_slabs, b_slabs, out_sizes, col_offsets, S, r_max,
                      rank_per_slot, scale_per_slot, token_to_slot, sorted_idx, slot_ids, counts, offsets, n_buckets,
                      scaling, dtype, impl, workspace, workspace_bytes, stream, 0);
}

int lora_b200_delta(void* delta, int64_t delta_ld, const void* x, int64_t x_ld, int32_t T, int32_t in_dim,
                    int32_t n_slices, const void* const* a_slabs, const void* const* b_slabs,
                    const int32_t* out_sizes, const int32_t* col_offsets, int32_t S, int32_t r_max,
                    const int32_t* rank_per_slot, const float* scale_per_slot,
                    const int32_t* token_to_slot, const int32_t* sorted_idx, const int32_t* slot_ids,
                    const int32_t* counts, const int32_t* offsets, int32_t n_buckets, float scaling,
                    int32_t dtype, int32_t impl, void* workspace, size_t workspace_bytes,
                    void* stream) {
  return add_or_delta(delta, delta_ld, x, x_ld, T, in_dim, n_slices, a_slabs, b_slabs, out_sizes, col_offsets, S, r_max,
                      rank_per_slot, scale_per_slot, token_to_slot, sorted_idx, slot_ids, counts, offsets, n_buckets,
                      scaling, dtype, impl, workspace, workspace_bytes, stream, 1);
}

int lora_b200_shrink(void* out, int32_t out_dtype, const void* x, int64_t x_ld, int32_t T,
                     int32_t in_dim, int32_t n_slices, const void* const* a_slabs, int32_t S,
                     int32_t r_max, const int32_t* token_to_slot, float scaling, int32_t dtype,
                     void* stream) {
  if (!valid_dtype(dtype) || !valid_dtype(out_dtype)) return fail(B200_LORA_EINVAL, "unknown dtype");
  if (out_dtype != dtype && out_dtype != B200_LORA_F32)
    return fail(B200_LORA_EUNSUPPORTED, "shrink output must have the input dtype or be f32");
  if (T < 0 || in_dim < 1 || S < 1 || r_max < 1) return fail(B200_LORA_EINVAL, "bad sizes");
  if (T == 0) return B200_LORA_OK;
  if (!out || !x || !token_to_slot) return fail(B200_LORA_EINVAL, "null out / x / token_to_slot");
  if (x_ld < in_dim) return fail(B200_LORA_EINVAL, "x_ld < in_dim");
  SliceTable st;
  if (int rc = fill_slices(st, n_slices, a_slabs, nullptr, nullptr, nullptr, true, false)) return rc;
  cudaStream_t st_ = static_cast<cudaStream_t>(stream);
  if (dtype == B200_LORA_BF16 && out_dtype == B200_LORA_BF16 && T >= kSgmvAutoMinTokens) {
    // prefill-sized bf16 batches: the tensor-core shrink (rows without adapter are written as zeros, as the
    // per-token kernel does); anything it does not take falls through to the per-token kernel
    SgmvProblem sp;
    sp.y = nullptr; sp.y_ld = 0; sp.x = x; sp.x_ld = x_ld; sp.T = T; sp.in_dim = in_dim; sp.S = S; sp.r_max = r_max;
    sp.st = st; sp.scale_per_slot = nullptr; sp.token_to_slot = token_to_slot; sp.scaling = scaling;
    if (sgmv_supported(sp, nullptr, true, false) && (reinterpret_cast<uintptr_t>(out) & 15u) == 0) {
      SgmvMaps sm;
      SgmvArgs sa;
      if (int rc = sgmv_prepare_tmp(sp, out, (uint64_t)st.n * T, true, false, &sm, &sa)) return rc;
      sa.zero_fill = 1;
      return sgmv_launch_shrink(sm, sa, st_);
    }
  }
#define B200_SHRINK(TT)                                                                              \
  (out_dtype == B200_LORA_F32 && dtype != B200_LORA_F32)                                             \
      ? launch_generic_shrink<TT, float>(out, x, x_ld, T, in_dim, st, S, r_max, token_to_slot, scaling, st_) \
      : launch_generic_shrink<TT, TT>(out, x, x_ld, T, in_dim, st, S, r_max, token_to_slot, scaling, st_)
  if (dtype == B200_LORA_BF16) return B200_SHRINK(__nv_bfloat16);
  if (dtype == B200_LORA_F16) return B200_SHRINK(__half);
  return launch_generic_shrink<float, float>(out, x, x_ld, T, in_dim, st, S, r_max, token_to_slot, scaling, st_);
#undef B200_SHRINK
}

int lora_b200_expand(void* y, int64_t y_ld, const void* tmp, int32_t tmp_dtype, int32_t T,
                     int32_t n_slices, const void* const* b_slabs, const int32_t* out_sizes,
                     const int32_t* col_offsets, int32_t S, int32_t r_max,
                     const int32_t* token_to_slot, int32_t add_inputs, int32_t dtype,
                     void* stream) {
  if (!valid_dtype(dtype) || !valid_dtype(tmp_dtype)) return fail(B200_LORA_EINVAL, "unknown dtype");
  if (tmp_dtype != dtype && tmp_dtype != B200_LORA_F32)
    return fail(B200_LORA_EUNSUPPORTED, "expand input must have the weight dtype or be f32");
  if (T < 0 || S < 1 || r_max < 1) return fail(B200_LORA_EINVAL, "bad sizes");
  if (T == 0) return B200_LORA_OK;
  if (!y || !tmp || !token_to_slot || !out_sizes || !col_offsets)
    return fail(B200_LORA_EINVAL, "null pointer argument");
  if (r_max > 2048) return fail(B200_LORA_EUNSUPPORTED, "r_max=%d > 2048", r_max);
  SliceTable st;
  if (int rc = fill_slices(st, n_slices, nullptr, b_slabs, out_sizes, col_offsets, false, true)) return rc;
  for (int s = 0; s < st.n; ++s)
    if (y_ld < (int64_t)st.col[s] + st.out[s]) return fail(B200_LORA_EINVAL, "y_ld smaller than slice end");
  cudaStream_t st_ = static_cast<cudaStream_t>(stream);
  if (dtype == B200_LORA_BF16 && tmp_dtype == B200_LORA_BF16 && add_inputs && T >= kSgmvAutoMinTokens) {
    // prefill-sized bf16 batches: the tensor-core expand (reduce-add tile kernel when the slices tile the
    // columns they cover in 64-column units, run-based kernel otherwise)
    int first = -1;
    for (int s = 0; s < st.n; ++s)
      if (st.out[s] > 0 && (first < 0 || st.col[s] < first)) first = st.col[s];
    bool dense = first >= 0;  // no zero-width slice in between: tmp is indexed by slice position
    for (int s = 0; s < st.n; ++s) dense = dense && st.out[s] > 0;
    if (dense && first % 8 == 0) {
      SgmvProblem sp;
      sp.y = static_cast<char*>(y) + (size_t)first * 2; sp.y_ld = y_ld; sp.x = nullptr; sp.x_ld = 0; sp.T = T; sp.in_dim = 0;
      sp.S = S; sp.r_max = r_max; sp.st = st; sp.scale_per_slot = nullptr; sp.token_to_slot = token_to_slot; sp.scaling = 1.0f;
      for (int s = 0; s < st.n; ++s) sp.st.col[s] -= first;
      if (sgmv_supported(sp, nullptr, false, true) && (reinterpret_cast<uintptr_t>(tmp) & 15u) == 0) {
        SgmvMaps sm;
        SgmvArgs sa;
        if (int rc = sgmv_prepare_tmp(sp, const_cast<void*>(tmp), (uint64_t)st.n * T, false, true, &sm, &sa)) return rc;
        if (tc_expand_fast_path_ok(sa)) {
          int n_total = 0;
          for (int s = 0; s < sa.n; ++s) n_total = std::max(n_total, sa.col[s] + sa.out[s]);
          GemmMaps gm;
          GemmArgs ga;
          if (int rc = tc_tile_prepare(sm, sa, nullptr, 0, n_total, nullptr, true, true, &gm, &ga, false, false)) return rc;
          return tc_tile_launch(gm, ga, st_);
        }
        return sgmv_launch_expand(sm, sa, st_);
      }
    }
  }
#define B200_EXPAND(TT)                                                                               \
  (tmp_dtype == B200_LORA_F32 && dtype != B200_LORA_F32)                                              \
      ? launch_generic_expand<TT, float>(y, y_ld, tmp, T, st, S, r_max, token_to_slot, add_inputs, st_) \
      : launch_generic_expand<TT, TT>(y, y_ld, tmp, T, st, S, r_max, token_to_slot, add_inputs, st_)
  if (dtype == B200_LORA_BF16) return B200_EXPAND(__nv_bfloat16);
  if (dtype == B200_LORA_F16) return B200_EXPAND(__half);
  return launch_generic_expand<float, float>(y, y_ld, tmp, T, st, S, r_max, token_to_slot, add_inputs, st_);
#undef B200_EXPAND
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// Prefill entry point for callers that cannot allocate device memory.
//
// The tensor-core prefill kernels keep the rank-r shrink result in scratch memory that
// lora_b200_add expects from its caller. Some callers have nowhere to get that from: code
// running inside an already captured or replaying CUDA graph, plug-ins that are handed
// input / output buffers by a host framework and are forbidden to call the allocator, and
// latency-critical loops that must not touch cudaMalloc (it synchronises the device). For them
// the same two kernels run on a fixed scratch array that is part of the library image.
//
// The array is one per GPU (every device that loads this library carries these bytes until
// the process exits) and is shared by every call on that GPU: it still holds the previous
// call's intermediate, and two calls that overlap on the GPU (different streams) would
// overwrite each other's intermediate. Nothing in it has to start at zero: each row that a
// call reads and uses was written by that same call's shrink kernel, rows of tokens without
// an adapter are read but masked out.
namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB: e.g. 3 slices x 8192 tokens x rank 64 in bf16 = 3 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void* g_static_scratch_addr[kMaxDevices] = {};

// Device address of the scratch array on the current device. In host code the array's name is
// only a handle of the runtime, not a device pointer, so the address is asked for once per
// device (with that device current) and remembered.
int static_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(B200_LORA_ECUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(B200_LORA_EUNSUPPORTED, "device ordinal %d not supported", dev);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(B200_LORA_ECUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
    g_static_scratch_addr[dev] = ptr;
  }
  *out = g_static_scratch_addr[dev];
  return B200_LORA_OK;
}

}  // namespace

extern "C" {

size_t lora_b200_static_scratch_bytes(void) { return kStaticScratchBytes; }

int lora_b200_add_prefill_noalloc(void* y, int64_t y_ld, const void* x, int64_t x_ld, int32_t T, int32_t in_dim,
                                  int32_t n_slices, const void* const* a_slabs, const void* const* b_slabs,
                                  const int32_t* out_sizes, const int32_t* col_offsets, int32_t S, int32_t r_max,
                                  const float* scale_per_slot, const int32_t* token_to_slot, float scaling,
                                  void* stream) {
  if (T < 0 || in_dim < 1 || S < 1 || r_max < 1)
    return fail(B200_LORA_EINVAL, "bad sizes T=%d in=%d S=%d r_max=%d", T, in_dim, S, r_max);
  if (T == 0) return B200_LORA_OK;
  if (y == nullptr || x == nullptr || token_to_slot == nullptr || out_sizes == nullptr || col_offsets == nullptr)
    return fail(B200_LORA_EINVAL, "null pointer argument");
  SliceTable st;
  if (int rc = fill_slices(st, n_slices, a_slabs, b_slabs, out_sizes, col_offsets, true, true)) return rc;
  int n_act = 0;
  int64_t width = 0;
  for (int s = 0; s < st.n; ++s) {
    n_act += st.out[s] > 0;
    width = width > (int64_t)st.col[s] + st.out[s] ? width : (int64_t)st.col[s] + st.out[s];
  }
  if (n_act == 0) return B200_LORA_OK;
  if (y_ld < width || x_ld < in_dim) return fail(B200_LORA_EINVAL, "row stride smaller than row");
  const size_t need = sgmv_workspace_bytes(T, n_act, r_max);
  if (need > kStaticScratchBytes)
    return fail(B200_LORA_EWORKSPACE,
                "batch needs %zu bytes of scratch (slices %d x tokens %d x rank %d, bf16) but the built-in scratch "
                "holds %zu; use lora_b200_add with caller-provided scratch",
                need, n_act, T, r_max, kStaticScratchBytes);
  SgmvProblem sp;
  sp.y = y; sp.y_ld = y_ld; sp.x = x; sp.x_ld = x_ld; sp.T = T; sp.in_dim = in_dim; sp.S = S; sp.r_max = r_max;
  sp.st = st; sp.scale_per_slot = scale_per_slot; sp.token_to_slot = token_to_slot; sp.scaling = scaling;
  void* scratch = nullptr;
  if (int rc = static_scratch_for_current_device(&scratch)) return rc;
  return prefill_add_launch(sp, scratch, kStaticScratchBytes, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
