// One-shot all-reduce of the row-parallel LoRA intermediate over peer memory (NVLink / NVSwitch).
//
// Row-parallel layers (o / down) shard lora_A on the input dimension, so every rank holds a partial
// tmp[n, T, r] (fp32) after its shrink. The reference lets that partial ride the [T, out] all-reduce
// of the base output (nanovllm_voxcpm/layers/lora.py:722-742); the smaller exchange is the sum of
// the [n, T, r] partials (r << out), after which every rank expands only its out/tp columns.
// This kernel is that exchange without a library collective: every rank PUSHES its partial into
// a slot of each peer's receive buffer with plain peer stores, publishes one flag per CTA chunk,
// waits (bounded) for the tp flags of its own chunk and adds the tp slots locally. One launch,
// one NVLink crossing per byte, no second synchronisation: ~3 us of latency where a library
// all-reduce of 128 KB costs 15-20 us.
//
// Memory (symmetric: same layout on every rank, peer pointers passed by the caller)
//   recv  : float[2][tp][capacity]   parity of the exchange counter x source rank
//   flags : int  [2][tp][kTpMaxCtas] value = exchange counter of the data in the slot
//   state : int  [2]                 local only: exchange counter, finished-CTA counter
// The receive buffer is double-buffered by the counter's parity: a rank can run at most one
// exchange ahead of its slowest peer (it needs that peer's flags of exchange e to finish e), so
// the slot of parity e & 1 is never rewritten before every rank has summed exchange e - 2.
// The counter lives in device memory and is advanced by the kernel itself, so a captured CUDA graph
// replays correctly. Ranks must issue the same sequence of exchanges. No multicast, no TMA: plain
// ld / st at system scope. Waits give up after a poll limit and raise the device status word.
#pragma once

#include "bgmv_fused.cuh"

namespace b200lora {

constexpr int kTpMaxRanks = 8;
constexpr int kTpMaxCtas = 64;
constexpr int kTpThreads = 256;
constexpr int kTpSpinLimit = 1 << 21;  // default poll limit of a system-scope load: about a second

// polls after which the wait for a peer's flag gives up (lora_b200_set_option, B200_LORA_OPT_PEER_POLL_LIMIT)
inline int& tp_spin_limit() {
  static int limit = kTpSpinLimit;
  return limit;
}

struct TpExchangeArgs {
  const float* partial;  // [count] this rank's partial sums
  float* out;            // [count] sum over the ranks (may alias partial)
  float* recv[kTpMaxRanks];
  int* flags[kTpMaxRanks];
  int* state;
  int rank, tp, count, capacity, n_cta;
  int spin_limit;  // polls of a peer's flag before the wait gives up
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kTpThreads) tp_allreduce_kernel(const TpExchangeArgs a) {
  __shared__ int gave_up;
  const int tid = threadIdx.x, cta = blockIdx.x;
  const int epoch = a.state[0] + 1;  // advanced by the last CTA to finish, read by all before that
  const int par = epoch & 1;
  if (tid == 0) gave_up = 0;
  const int vec = a.count >> 2;  // float4 units
  const int per = (vec + a.n_cta - 1) / a.n_cta;
  const int lo = min(cta * per, vec), hi = min(lo + per, vec);
  const size_t slot = ((size_t)par * a.tp + a.rank) * (size_t)a.capacity;
  const float4* src = reinterpret_cast<const float4*>(a.partial);

  // 1. push this CTA's chunk into slot [par][rank] of every rank (own rank included)
  for (int k = 0; k < a.tp; ++k) {
    const int peer = (a.rank + 1 + k) % a.tp;  // start with the neighbour: ranks do not all hit rank 0 first
    float4* dst = reinterpret_cast<float4*>(a.recv[peer] + slot);
    for (int i = lo + tid; i < hi; i += kTpThreads) dst[i] = src[i];
  }
  // 2. publish: one flag per (source rank, CTA chunk) on every rank. The CTA barrier orders every
  //    thread's stores before the publishing threads, whose release at system scope is cumulative.
  __syncthreads();
  if (tid < a.tp) st_release_sys(a.flags[tid] + ((size_t)par * a.tp + a.rank) * kTpMaxCtas + cta, epoch);
  // 3. wait for the same chunk of every source rank (bounded)
  if (tid < a.tp) {
    const int* f = a.flags[a.rank] + ((size_t)par * a.tp + tid) * kTpMaxCtas + cta;
    int it = 0;
    while (ld_acquire_sys(f) != epoch) {
      if (++it >= a.spin_limit) { gave_up = 1; break; }
    }
  }
  __syncthreads();
  // 4. add the tp slots of the local receive buffer
  const float* base = a.recv[a.rank] + (size_t)par * a.tp * (size_t)a.capacity;
  float4* out = reinterpret_cast<float4*>(a.out);
  for (int i = lo + tid; i < hi; i += kTpThreads) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < a.tp; ++r) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(base + (size_t)r * a.capacity) + i);  // L2: peers wrote it
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    out[i] = s;
  }
  // 5. the last CTA of this launch advances the exchange counter for the next launch of the stream
  __syncthreads();
  if (tid == 0) {
    if (gave_up) atomicOr(&g_b200_status, kStatusPeerWaitGaveUp);
    __threadfence();
    if (atomicAdd(&a.state[1], 1) == a.n_cta - 1) {
      a.state[1] = 0;
      __threadfence();
      a.state[0] = epoch;
    }
  }
}

inline size_t tp_exchange_bytes(int tp, int capacity) {
  return (size_t)2 * tp * capacity * sizeof(float) + (size_t)2 * tp * kTpMaxCtas * sizeof(int) + 64;
}

// Byte offsets of the three regions inside one rank's symmetric buffer of tp_exchange_bytes().
inline size_t tp_flags_offset(int tp, int capacity) { return (size_t)2 * tp * capacity * sizeof(float); }
inline size_t tp_state_offset(int tp, int capacity) { return tp_flags_offset(tp, capacity) + (size_t)2 * tp * kTpMaxCtas * sizeof(int); }

inline int tp_allreduce_launch(const float* partial, float* out, int count, void* const* peer_buffers, int rank, int tp,
                               int capacity, cudaStream_t stream) {
  if (tp < 1 || tp > kTpMaxRanks || rank < 0 || rank >= tp) return fail(B200_LORA_EINVAL, "tp exchange: rank %d of %d", rank, tp);
  if (count < 0 || count > capacity || (count & 3) || (capacity & 3))
    return fail(B200_LORA_EINVAL, "tp exchange: count %d must be a multiple of 4 and <= capacity %d", count, capacity);
  if (count == 0) return B200_LORA_OK;
  if (partial == nullptr || out == nullptr || peer_buffers == nullptr) return fail(B200_LORA_EINVAL, "tp exchange: null pointer");
  TpExchangeArgs a = {};
  a.partial = partial; a.out = out; a.rank = rank; a.tp = tp; a.count = count; a.capacity = capacity;
  for (int r = 0; r < tp; ++r) {
    if (peer_buffers[r] == nullptr) return fail(B200_LORA_EINVAL, "tp exchange: null peer buffer %d", r);
    uint8_t* b = static_cast<uint8_t*>(peer_buffers[r]);
    a.recv[r] = reinterpret_cast<float*>(b);
    a.flags[r] = reinterpret_cast<int*>(b + tp_flags_offset(tp, capacity));
  }
  a.state = reinterpret_cast<int*>(static_cast<uint8_t*>(peer_buffers[rank]) + tp_state_offset(tp, capacity));
  a.n_cta = std::max(1, std::min(kTpMaxCtas, (count * 4 + 16383) / 16384));
  a.spin_limit = tp_spin_limit();
  tp_allreduce_kernel<<<a.n_cta, kTpThreads, 0, stream>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_LORA_ECUDA, "tp_allreduce_kernel launch: %s", cudaGetErrorString(e));
  return B200_LORA_OK;
}

}  // namespace b200lora
