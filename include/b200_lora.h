/*
 * b200_lora.h - C ABI of the B200 (sm_100a) batched multi-LoRA linear library.
 *
 * Every entry point takes plain pointers and sizes; no C++ or torch types cross
 * this boundary. Pointers documented "device" are CUDA device addresses owned by
 * the caller, pointers documented "host" are ordinary host arrays read during the
 * call. `stream` is a `cudaStream_t` passed as `void*` (NULL = legacy default
 * stream). All launches are asynchronous on that stream and allocate nothing.
 *
 * Return value: 0 on success, a negative B200_LORA_E* code otherwise, in which
 * case nothing was launched and `lora_b200_last_error()` returns a message for the
 * calling thread.
 *
 * Reference interfaces are cited by their path inside the a710128/nanovllm-voxcpm
 * project (e.g. nanovllm_voxcpm/lora.py:43-54).
 *
 * Slab layout (nanovllm_voxcpm/layers/lora.py:289-298,507-511,703-705,828-829):
 *   lora_A slice  [S, r_max, in ]  row-major, contiguous
 *   lora_B slice  [S, out_s, r_max] row-major, contiguous
 * where S = number of adapter slots and r_max the slab rank; rows/columns beyond
 * a slot's effective rank hold zeros.
 */
#ifndef B200_LORA_H_
#define B200_LORA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_LORA_ABI_VERSION 1

/* element types of x / y / slabs */
#define B200_LORA_BF16 0
#define B200_LORA_F16 1
#define B200_LORA_F32 2

/* kernel selection for lora_b200_add (`impl`) */
#define B200_LORA_IMPL_AUTO 0    /* choose by shape */
#define B200_LORA_IMPL_GENERIC 1 /* one CTA per token, any dtype / shape / stride */
#define B200_LORA_IMPL_BGMV 2    /* fused decode kernel: cluster per slot bucket, bulk-copy ring + mma */
#define B200_LORA_IMPL_SGMV 3    /* prefill kernels: tcgen05 shrink + tcgen05 expand, scratch from `workspace` */

/* error codes */
#define B200_LORA_OK 0
#define B200_LORA_EINVAL (-1)      /* bad argument (shape, alignment, null pointer) */
#define B200_LORA_EUNSUPPORTED (-2) /* requested impl cannot run this shape / dtype */
#define B200_LORA_ECUDA (-3)       /* CUDA runtime / driver error at launch */
#define B200_LORA_EWORKSPACE (-4)  /* workspace too small */

#define B200_LORA_MAX_SLICES 4

/* ABI version of the loaded library (== B200_LORA_ABI_VERSION it was built with).
 * No counterpart in the reference; lets a binding refuse a stale build. */
int lora_b200_version(void);

/* Message for the last non-zero return on this thread (never NULL). */
const char* lora_b200_last_error(void);

/*
 * y[t, col_offsets[s] : col_offsets[s]+out_sizes[s]] +=
 *        scaling * scale_per_slot[slot_t] * (x[t] . A_s[slot_t]^T) . B_s[slot_t]^T
 * for every token t with slot_t = token_to_slot[t] >= 0, in place. Rows with
 * slot_t < 0 are never read or written (their bits are preserved).
 *
 * Replaces `LoRABackend.add_lora` / `_VendoredTritonPunicaBackend.add_lora`
 * (nanovllm_voxcpm/lora.py:43-54, :241-381), i.e. `lora_shrink` + `lora_expand`
 * (nanovllm_voxcpm/lora_ops/triton_ops/lora_shrink_op.py:257-341,
 *  lora_expand_op.py:94-170) with add_inputs=True, all slices in one call.
 *
 *  y, x            device; [T, *] matrices with row strides y_ld / x_ld (elements),
 *                  unit column stride.
 *  a_slabs,b_slabs host arrays of n_slices device pointers (layout above).
 *  out_sizes       host[n_slices]; width of each slice (0 = slice skipped).
 *  col_offsets     host[n_slices]; first y column of each slice.
 *  rank_per_slot   device int32[S] or NULL: effective rank per slot (an optimisation
 *                  only: slab padding is zero, results are identical).
 *  scale_per_slot  device float[S] or NULL (= 1).
 *  token_to_slot   device int32[T]; slot id or -1        (LoRAMetadata.token_to_slot,
 *                  nanovllm_voxcpm/lora.py:18-37).
 *  sorted_idx      device int32[<=T] or NULL: token rows grouped by bucket
 *  slot_ids        device int32[n_buckets] or NULL: slot id per bucket (-1 = unused)
 *  counts          device int32[n_buckets] or NULL: tokens per bucket
 *  offsets         device int32[n_buckets+1] or NULL: bucket start in sorted_idx
 *                  (the reference's token_indices_sorted_by_slot / active_slot_ids /
 *                  num_tokens_per_slot / slot_start_offsets; any of its three
 *                  conventions: eager plan, graph buffers with a leading -1 bucket,
 *                  vLLM-style with a counted -1 bucket). With the bucket arrays NULL
 *                  only the generic kernel can run.
 *  workspace       device scratch for B200_LORA_IMPL_SGMV (see lora_b200_workspace_bytes); may be
 *                  NULL otherwise. With B200_LORA_IMPL_AUTO the prefill kernels are chosen only
 *                  when enough scratch is passed.
 */
int lora_b200_add(void* y, int64_t y_ld, const void* x, int64_t x_ld, int32_t T, int32_t in_dim,
                  int32_t n_slices, const void* const* a_slabs, const void* const* b_slabs,
                  const int32_t* out_sizes, const int32_t* col_offsets, int32_t S, int32_t r_max,
                  const int32_t* rank_per_slot, const float* scale_per_slot,
                  const int32_t* token_to_slot, const int32_t* sorted_idx, const int32_t* slot_ids,
                  const int32_t* counts, const int32_t* offsets, int32_t n_buckets, float scaling,
                  int32_t dtype, int32_t impl, void* workspace, size_t workspace_bytes,
                  void* stream);

/*
 * delta[t, cols] = scaling * scale_per_slot[slot_t] * (x[t] . A_s[slot_t]^T) . B_s[slot_t]^T for rows with an
 * adapter, and -0.0 (sign bit only) over the slices' columns of every other row; delta is written, never read.
 * Arguments as lora_b200_add. For a caller that runs the LoRA part BEFORE the base GEMM and lets the GEMM
 * accumulate into the same buffer (beta = 1): x + (-0.0) == x, so rows without adapter end up bit-identical to
 * the plain base result, and the launch no longer waits for the GEMM (under programmatic dependent launch its
 * weight fetch overlaps whatever kernel of the caller runs before it). Decode batches take the fused kernel in
 * overwrite mode; other shapes fill with -0.0 and add. No counterpart in the reference, which always adds after
 * the base GEMM (nanovllm_voxcpm/layers/lora.py:341-366).
 */
int lora_b200_delta(void* delta, int64_t delta_ld, const void* x, int64_t x_ld, int32_t T, int32_t in_dim,
                    int32_t n_slices, const void* const* a_slabs, const void* const* b_slabs,
                    const int32_t* out_sizes, const int32_t* col_offsets, int32_t S, int32_t r_max,
                    const int32_t* rank_per_slot, const float* scale_per_slot,
                    const int32_t* token_to_slot, const int32_t* sorted_idx, const int32_t* slot_ids,
                    const int32_t* counts, const int32_t* offsets, int32_t n_buckets, float scaling,
                    int32_t dtype, int32_t impl, void* workspace, size_t workspace_bytes,
                    void* stream);

/*
 * y = x . W^T (+ bias) + LoRA delta in one pass over y: the base GEMM runs on the tensor cores
 * and, for every 128-row block whose rows use one adapter slot, the delta tmp . B^T is
 * accumulated into the same TMEM accumulator before the single store of y (blocks with mixed
 * slots get their delta from the run-based expand kernel afterwards).
 *
 * Replaces the `F.linear` + `add_lora` pair of the layer forwards
 * (nanovllm_voxcpm/layers/lora.py:341-366, 547-570, 723-738, 832-848).
 *  weight      device; [out_total, in] bf16, row pitch w_ld elements
 *  bias        device bf16[out_total] or NULL
 *  token_to_slot NULL or n_slices == 0: plain linear, no adapter work
 *  workspace   device scratch of lora_b200_workspace_bytes(T, active slices, r_max) bytes
 *              (may be NULL for a plain linear)
 * bf16 only; in % 64 == 0; r_max in {16, 32, 64}. Other arguments as in lora_b200_add.
 */
int lora_b200_linear_lora(void* y, int64_t y_ld, const void* x, int64_t x_ld, int32_t T, int32_t in_dim,
                          const void* weight, int64_t w_ld, int32_t out_total, const void* bias,
                          int32_t n_slices, const void* const* a_slabs, const void* const* b_slabs,
                          const int32_t* out_sizes, const int32_t* col_offsets, int32_t S,
                          int32_t r_max, const float* scale_per_slot, const int32_t* token_to_slot,
                          float scaling, void* workspace, size_t workspace_bytes, void* stream);

/* Bytes of device scratch that B200_LORA_IMPL_SGMV needs for a batch of T tokens (the
 * [n_slices, T, r_max] shrink result in bf16, plus alignment slack). The reference allocates this
 * intermediate itself on every call (nanovllm_voxcpm/lora.py:302). */
size_t lora_b200_workspace_bytes(int32_t T, int32_t n_slices, int32_t r_max);

/*
 * out[s, t, 0:r_max] = scaling * x[t] . A_s[slot_t]^T for slot_t >= 0, and 0 for
 * rows with slot_t < 0 (the reference zero-fills the buffer first,
 * lora_shrink_op.py:229,295).
 *
 * Replaces `lora_shrink` (nanovllm_voxcpm/lora_ops/triton_ops/lora_shrink_op.py:257-341).
 *  out        device; [n_slices, T, r_max] contiguous; element type out_dtype
 *             (B200_LORA_F32 is accepted for any input dtype: used by the
 *             row-parallel [T, r] all-reduce).
 */
int lora_b200_shrink(void* out, int32_t out_dtype, const void* x, int64_t x_ld, int32_t T,
                     int32_t in_dim, int32_t n_slices, const void* const* a_slabs, int32_t S,
                     int32_t r_max, const int32_t* token_to_slot, float scaling, int32_t dtype,
                     void* stream);

/*
 * y[t, offset_start + sum(out_sizes[:s]) + c] (+)= tmp[s, t, :] . B_s[slot_t][c, :]
 * for slot_t >= 0; `add_inputs` = 0 overwrites instead of accumulating.
 *
 * Replaces `lora_expand` (nanovllm_voxcpm/lora_ops/triton_ops/lora_expand_op.py:94-170).
 *  tmp        device; [n_slices, T, r_max] contiguous, element type tmp_dtype.
 */
int lora_b200_expand(void* y, int64_t y_ld, const void* tmp, int32_t tmp_dtype, int32_t T,
                     int32_t n_slices, const void* const* b_slabs, const int32_t* out_sizes,
                     const int32_t* col_offsets, int32_t S, int32_t r_max,
                     const int32_t* token_to_slot, int32_t add_inputs, int32_t dtype,
                     void* stream);

/*
 * Prefill multi-LoRA add for callers that cannot allocate device memory (code running
 * under CUDA-graph capture or replay, plug-ins that only receive input / output buffers
 * from their host framework, latency-critical loops that must stay away from cudaMalloc).
 * Same result as lora_b200_add with B200_LORA_IMPL_SGMV, but the rank-r intermediate lives
 * in a fixed array inside the library instead of caller-provided scratch; no allocation of
 * any kind happens in this call. It has no counterpart in the reference, whose backend
 * allocates that intermediate with torch.empty on every call.
 *
 * Limits and rules:
 *  - the batch must fit the built-in scratch: lora_b200_workspace_bytes(T, active slices,
 *    r_max) <= lora_b200_static_scratch_bytes() (8 MiB); larger batches are rejected with
 *    B200_LORA_EWORKSPACE and nothing is launched;
 *  - bf16 only, shapes as for B200_LORA_IMPL_SGMV (r_max 16/32/64, in % 64 == 0);
 *  - the first call on each GPU looks up the array's device address (cudaGetSymbolAddress,
 *    which may load the module): make that first call outside of any stream capture;
 *  - there is one array per GPU, shared by all calls and still holding the previous call's
 *    intermediate; calls that may overlap on the GPU (different streams without ordering)
 *    race on it. Calls on one stream are safe.
 * Arguments have the meaning they have in lora_b200_add.
 */
int lora_b200_add_prefill_noalloc(void* y, int64_t y_ld, const void* x, int64_t x_ld, int32_t T,
                                  int32_t in_dim, int32_t n_slices, const void* const* a_slabs,
                                  const void* const* b_slabs, const int32_t* out_sizes,
                                  const int32_t* col_offsets, int32_t S, int32_t r_max,
                                  const float* scale_per_slot, const int32_t* token_to_slot,
                                  float scaling, void* stream);

/* Size in bytes of the built-in scratch used by lora_b200_add_prefill_noalloc. No counterpart in
 * the reference. */
size_t lora_b200_static_scratch_bytes(void);

/*
 * Adapter admission in one launch. `staging` is the device copy of ONE packed buffer: `n_desc`
 * 64-byte descriptors, then the payload tensors they point into (byte offsets from the start of
 * the buffer). A descriptor either fills one slab region of the slot,
 *     dst[i, j] = (i < src_rows && j < src_cols) ? round(float(src[i * src_ld + j]) * scale) : 0
 * over dst_rows x dst_cols (the slot's [r_max, in] block of lora_A, or its [out, r_max] block of
 * lora_B with scale = the adapter's scaling), or writes one int32 / float scalar (the slot's entries
 * of effective_lora_rank / lora_scaling / lora_base_scaling). Layout of a descriptor, little endian:
 *     u64 dst; i64 src_offset; i32 kind (0 region, 1 int32 scalar, 2 floating scalar of dst_dtype); i32 dst_rows, dst_cols;
 *     i32 src_rows, src_cols, src_ld; i32 src_dtype, dst_dtype (B200_LORA_BF16 / F16 / F32);
 *     f32 scale (kind 2: the value); i32 ivalue (kind 1: the value); 8 bytes padding.
 * `max_elems` = largest dst_rows * dst_cols of the table.
 * Replaces the per-module loop of `_load_lora_slot` + `set_slot_lora`
 * (nanovllm_voxcpm/engine/model_runner.py:389-420, nanovllm_voxcpm/layers/lora.py:395-417): same slab
 * contents, one host->device copy and one kernel instead of several per module.
 */
int lora_b200_load_slot(const void* staging, int32_t n_desc, int64_t max_elems, void* stream);

/*
 * Memory-bound glue of a decoder layer around the four projections (bf16 / fp16, rows 16-byte aligned,
 * widths multiples of 8), one launch each, the row read once and written once.
 *
 * lora_b200_glue_add_rmsnorm: hidden = residual + x (rounded to dtype), normed = hidden * rsqrt(mean(hidden^2)
 * + eps) * weight, statistics in fp32, one rounding of the result. residual NULL: plain rms_norm of x.
 * hidden_out NULL: the sum is not stored; it may alias residual or x. norm_of_rounded_sum = 1: the norm
 * reads the rounded sum (`hidden = residual + sublayer(...)` followed by `RMSNorm.rms_forward`,
 * nanovllm_voxcpm/models/voxcpm2/model.py:291-297, layers/layernorm.py:18-22); 0: the fp32 sum
 * (`RMSNorm.add_rms_forward`, layers/layernorm.py:24-32). hidden <= 4096.
 *
 * lora_b200_glue_rope_kv_store: qkv [T, (num_heads + 2 num_kv_heads) * head_dim] = q | k | v per row. Rotates
 * every q and k head in place, y = x * cos[pos] + rotate_half(x) * sin[pos] with fp32 products and sum rounded
 * separately (`apply_rotary_emb`, models/voxcpm2/model_utils_rope.py:50-63, called from
 * `MiniCPMLongRoPE.forward`, models/voxcpm2/model.py:81-94), cos / sin tables [max_position, table_dim] of
 * table_dtype with table_dim = head_dim (the reference's cache) or head_dim / 2, positions clamped to the
 * table; then copies the rotated k row and the v row to k_cache / v_cache [slots, num_kv_heads * head_dim] at
 * slot_mapping[t], skipping -1 (`store_kvcache`, layers/attention.py:10-49). positions / tables all NULL: no
 * rotation (use_rope = False); caches NULL: no store. head_dim must be a multiple of 16.
 *
 * lora_b200_glue_silu_mul: out[t, j] = silu(gate_up[t, j]) * gate_up[t, intermediate + j] in fp32, one rounding
 * (`SiluAndMul`, layers/activation.py:11-14).
 */
int lora_b200_glue_add_rmsnorm(void* normed, int64_t normed_ld, void* hidden_out, int64_t hidden_ld, const void* x,
                               int64_t x_ld, const void* residual, int64_t residual_ld, const void* weight, int32_t T,
                               int32_t hidden, float eps, int32_t norm_of_rounded_sum, int32_t dtype, void* stream);
int lora_b200_glue_rope_kv_store(void* qkv, int64_t qkv_ld, int32_t T, int32_t num_heads, int32_t num_kv_heads,
                                 int32_t head_dim, const int64_t* positions, const void* cos_table, const void* sin_table,
                                 int32_t table_dim, int32_t table_dtype, int32_t max_position, void* k_cache, void* v_cache,
                                 const int32_t* slot_mapping, int32_t dtype, void* stream);
int lora_b200_glue_silu_mul(void* out, int64_t out_ld, const void* gate_up, int64_t gate_up_ld, int32_t T,
                            int32_t intermediate, int32_t dtype, void* stream);

/* conventions of lora_b200_build_metadata */
#define B200_LORA_META_GRAPH 0  /* fixed buckets [-1, 0 .. S-1], bucket 0 always empty (CUDA-graph buffers) */
#define B200_LORA_META_KERNEL 1 /* compact ids incl. the -1 bucket with its rows (LoRAKernelMeta.prepare_tensors) */
#define B200_LORA_META_EAGER 2  /* compact ids of the slots >= 0 that occur (eager batch plan) */

/*
 * Builds the step's index metadata from token_to_slot on the device, in one launch: the stable
 * order of token rows by slot, rows per bucket and bucket start offsets. Same integers, bit for
 * bit, as the reference builds on the host with loops over the tokens and then copies over:
 * `build_lora_batch_plan_from_token_to_slot` (nanovllm_voxcpm/engine/lora_manager.py:77-111) for
 * EAGER, `_copy_lora_domain_to_graph_vars` (engine/model_runner.py:774-797) for GRAPH,
 * `LoRAKernelMeta.prepare_tensors` (lora_ops/triton_ops/lora_kernel_metadata.py:47-67) for KERNEL.
 *  token_to_slot device int32[T]; ids outside [-1, S) count as -1 and are reported in info[2]
 *  sorted_idx    device int32[>= T]; GRAPH / EAGER write the rows with an adapter (the tail keeps
 *                its old content), KERNEL writes all T rows
 *  slot_ids      device int32[S+1]; may be NULL for GRAPH (the ids are the constants -1 .. S-1)
 *  counts        device int32[S+1];  offsets device int32[S+2]
 *  info          device int32[3] or NULL: buckets in use, rows with an adapter, rows with a bad id
 * T <= 16384, 1 <= S <= 4095.
 */
int lora_b200_build_metadata(const int32_t* token_to_slot, int32_t T, int32_t S, int32_t convention,
                             int32_t* sorted_idx, int32_t* slot_ids, int32_t* counts, int32_t* offsets,
                             int32_t* info, void* stream);

/*
 * Tensor-parallel exchange of the row-parallel LoRA intermediate: out[i] = sum over the tp ranks of
 * partial[i], in ONE kernel over peer memory (each rank pushes its partial into every peer's receive
 * buffer with plain stores over NVLink, publishes per-chunk flags, waits - bounded - for its peers'
 * and adds). It stands where the reference has no separate collective: there the partial LoRA delta
 * rides the [T, out] all-reduce of the base output (nanovllm_voxcpm/layers/lora.py:722-742); summing
 * the [n, T, r] shrink results instead lets every rank expand only its out/tp columns of lora_B.
 *  partial, out  device float[count] (may alias); count % 4 == 0, count <= capacity
 *  peer_buffers  host array of tp device pointers: rank r's symmetric buffer of
 *                lora_b200_tp_exchange_bytes(tp, capacity) bytes, zero-filled once, mapped into
 *                this process (CUDA IPC / symmetric memory); entry [rank] is the local one
 * Every rank must issue the same sequence of calls. The exchange counter lives in the buffer, so
 * a captured CUDA graph replays correctly. A wait that gives up sets bit 2 of the device status.
 */
int lora_b200_tp_allreduce(const float* partial, float* out, int32_t count, void* const* peer_buffers,
                           int32_t rank, int32_t tp, int32_t capacity, void* stream);
size_t lora_b200_tp_exchange_bytes(int32_t tp, int32_t capacity);

/*
 * Row-parallel (o / down) multi-LoRA add of one tensor-parallel rank:
 *   tmp = scaling * x_shard . A_shard^T      (bucket kernel in shrink-only form, fp32 [n, T, r_max])
 *   tmp = sum of tmp over the tp ranks       (lora_b200_tp_allreduce over peer memory)
 *   y_partial[:, col_offsets ..] += tmp . B_shard^T   (bucket kernel in expand-only form)
 * with lora_A sharded on the input dim and lora_B on the OUTPUT dim, so each rank reads 1/tp of B and
 * the base output's own [T, out] all-reduce assembles the delta exactly once. The reference keeps B
 * whole on every rank and lets the partial delta ride that all-reduce
 * (nanovllm_voxcpm/layers/lora.py:714-742).
 *  x, a_slabs   this rank's input shard [T, in/tp] and lora_A shards [S, r_max, in/tp]
 *  b_slabs      this rank's lora_B shards [S, out_s/tp, r_max]; col_offsets: their first y column
 *  tmp          device float[n_slices * T * r_max] scratch (n_slices * T * r_max % 4 == 0)
 *  peer_buffers, rank, tp, capacity   as lora_b200_tp_allreduce (ignored for tp == 1)
 * Other arguments as lora_b200_add (no zero-width slices). bf16 with bucket arrays runs the fused decode
 * kernel's two halves; everything else one-CTA-per-token kernels.
 */
int lora_b200_shrink_allreduce_expand(void* y, int64_t y_ld, const void* x, int64_t x_ld, int32_t T, int32_t in_dim,
                                      int32_t n_slices, const void* const* a_slabs, const void* const* b_slabs,
                                      const int32_t* out_sizes, const int32_t* col_offsets, int32_t S, int32_t r_max,
                                      const int32_t* rank_per_slot, const float* scale_per_slot,
                                      const int32_t* token_to_slot, const int32_t* sorted_idx, const int32_t* slot_ids,
                                      const int32_t* counts, const int32_t* offsets, int32_t n_buckets, float scaling,
                                      int32_t dtype, float* tmp, void* const* peer_buffers, int32_t rank, int32_t tp,
                                      int32_t capacity, void* stream);

/* Tuning knobs of the fused decode kernel (process-wide, read at launch time). */
#define B200_LORA_OPT_CLUSTER 1 /* CTAs per slot bucket: 1, 2, 4, 8; 0 = choose from n_buckets */
#define B200_LORA_OPT_PDL 2     /* 1 = launch with programmatic stream serialization (default), 0 = off */
#define B200_LORA_OPT_RING_KB 3 /* cap of the shared-memory stage ring in KB, 0 = as large as fits */
#define B200_LORA_OPT_PEER_POLL_LIMIT 7 /* tensor-parallel exchange: polls of a peer's flag after which the wait gives up and bit 2 of the device status word is set; 0 = default (about a second) */
#define B200_LORA_OPT_KSPLIT 6 /* fused decode kernel: 1 = deal the K parts of long input rows (>= 1024 columns per CTA of a cluster) over the cluster (default), 0 = always split the rank rows */

/* Sets a tuning knob; returns 0, or B200_LORA_EINVAL for an unknown key / value.
 * No counterpart in the reference (its tile configs are static tables,
 * nanovllm_voxcpm/lora_ops/triton_ops/utils.py:119-150). */
int lora_b200_set_option(int32_t key, int32_t value);

/* Reads (and, if `reset` != 0, clears) the status word of the current device into
 * *status: 0 = no kernel ever gave up a bounded wait. Synchronises the device; meant
 * for tests and health checks, not for the hot path. No counterpart in the reference. */
int lora_b200_device_status(int32_t* status, int32_t reset);

#ifdef B200_TRACE
/* Tuning build only (the library compiled with -DB200_TRACE): copies `n_values` (<= 1024 * 32) SM-clock timestamps
 * of the last fused-decode launch - 32 phase marks for each of the first 1024 slot buckets, taken by the first CTA of
 * the bucket's cluster - into `out`. No counterpart in the reference. */
int lora_b200_debug_trace(long long* out, int32_t n_values);
#endif

#ifdef __cplusplus
}
#endif
#endif /* B200_LORA_H_ */
