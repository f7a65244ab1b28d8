"""Peer-memory exchange of the row-parallel LoRA intermediate (tensor parallelism).

``TpExchange`` owns one symmetric buffer per rank (``torch.distributed._symmetric_memory``: the same
allocation mapped into every rank of the group, peers reachable over NVLink) and sums fp32 partials
over the tensor-parallel group with ``lora_b200_tp_allreduce``: one kernel per exchange, no library
collective. It serves ``LoRARowParallelLinear`` in ``lora_tp_mode="peer_exchange"``, where each rank
shrinks on its input shard, the ``[n, T, r]`` partials are summed here, and each rank expands only
its ``out / tp`` columns of ``lora_B``; the base output's own ``[T, out]`` all-reduce
(``nanovllm_voxcpm/layers/lora.py:722-742``) then assembles the full delta exactly once.

Every rank must issue the same sequence of exchanges. Multicast is not used: the kernel issues plain peer
stores, and the symmetric allocation is made with ``TORCH_SYMM_MEM_DISABLE_MULTICAST=1`` (set here before
torch's symmetric memory is first imported), so that the buffer is never bound to an NVLink multicast object -
a rank that dies while its memory is bound to one can fault its peers.
"""

from __future__ import annotations

import os

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

import torch
import torch.distributed as dist

from . import _native as N


class TpExchange:
    def __init__(self, capacity: int, group=None, device: torch.device | None = None):
        """``capacity``: largest number of fp32 values of one exchange (rounded up to a multiple of 4)."""
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.tp = dist.get_world_size(self.group)
        self.capacity = (int(capacity) + 3) & ~3
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        nbytes = int(N.lib().lora_b200_tp_exchange_bytes(self.tp, self.capacity))
        self._buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self._buffer.zero_()
        torch.cuda.synchronize(self.device)
        self._handle = symm_mem.rendezvous(self._buffer, group=self.group)
        mc = getattr(self._handle, "multicast_ptr", 0)
        if mc not in (0, None):
            raise RuntimeError("the exchange buffer was bound to an NVLink multicast object; set "
                               "TORCH_SYMM_MEM_DISABLE_MULTICAST=1 before torch.distributed._symmetric_memory is imported")
        self._peers = (N.c_void_p * self.tp)(*[int(p) for p in self._handle.buffer_ptrs])
        #: fp32 intermediate of shrink_allreduce_expand: owned here, fixed size, so an address captured in a
        #: CUDA graph stays valid however the shared scratch of other calls grows
        self._tmp = torch.empty(self.capacity * 4 + 256, dtype=torch.uint8, device=self.device)
        dist.barrier(self.group)  # every rank's buffer is zeroed and mapped before the first push

    def all_reduce_(self, partial: torch.Tensor) -> torch.Tensor:
        """In place: ``partial`` (fp32, contiguous, numel % 4 == 0) becomes the sum over the group."""
        N.require_cuda(partial)
        if partial.dtype != torch.float32 or not partial.is_contiguous():
            raise ValueError("the exchanged partial must be a contiguous float32 tensor")
        with N.on_device(partial.device):
            N.check(N.lib().lora_b200_tp_allreduce(partial.data_ptr(), partial.data_ptr(), partial.numel(), self._peers,
                                                   self.rank, self.tp, self.capacity, N.current_stream(partial.device)))
        return partial

    def row_parallel_add(self, y, x, a_slabs, b_slabs, out_sizes, col_offsets, metadata, scaling: float = 1.0, *,
                         rank_per_slot=None, scale_per_slot=None) -> None:
        """Shrink on this rank's input shard, sum the ``[n, T, r]`` partials over the group through peer
        memory, expand this rank's output shard of ``lora_B`` into the partial ``y``: one C call, three
        launches, no library collective."""
        shrink_allreduce_expand(y, x, a_slabs, b_slabs, out_sizes, col_offsets, metadata, scaling,
                                rank_per_slot=rank_per_slot, scale_per_slot=scale_per_slot, exchange=self)


def shrink_allreduce_expand(y, x, a_slabs, b_slabs, out_sizes, col_offsets, metadata, scaling: float = 1.0, *,
                            rank_per_slot=None, scale_per_slot=None, exchange: TpExchange | None = None) -> None:
    """One ``lora_b200_shrink_allreduce_expand`` call; ``exchange=None`` is the single-rank form (no peers)."""
    from .lora import _as_3d, _i32, scratch_for

    N.require_cuda(y, x, *a_slabs, *b_slabs, metadata.token_to_slot)
    if x.dim() != 2 or y.dim() != 2 or x.stride(1) != 1 or y.stride(1) != 1:
        raise ValueError("x and y must be 2D with unit column stride")
    a_slabs = [_as_3d(a) for a in a_slabs]
    b_slabs = [_as_3d(b) for b in b_slabs]
    T, in_dim = x.shape
    S, r_max, _ = a_slabs[0].shape
    n = len(a_slabs)
    peers, rank, tp, capacity = None, 0, 1, 4
    if exchange is not None:
        peers, rank, tp, capacity = exchange._peers, exchange.rank, exchange.tp, exchange.capacity
        if tp > 1 and n * T * r_max > capacity:
            raise ValueError(f"exchange of {n * T * r_max} values exceeds the capacity {capacity} of this TpExchange")
    tts, srt, cnt, off, ids, _, _ = metadata.as_kernel_metadata(T)
    n_buckets = 0
    if srt is not None and ids is not None and cnt is not None and off is not None:
        n_buckets = min(ids.numel(), cnt.numel(), off.numel() - 1)
        if metadata.num_active_loras > 0:
            n_buckets = min(n_buckets, metadata.num_active_loras)
    if n_buckets <= 0:
        srt = ids = cnt = off = None
        n_buckets = 0
    tmp = exchange._tmp if exchange is not None and n * T * r_max <= exchange.capacity else scratch_for(x.device, n * T * r_max * 4 + 256)
    tmp_ptr = (tmp.data_ptr() + 255) & ~255
    with N.on_device(x.device):
        N.check(N.lib().lora_b200_shrink_allreduce_expand(
            y.data_ptr(), y.stride(0), x.data_ptr(), x.stride(0), T, in_dim, n, N.ptr_array(a_slabs), N.ptr_array(b_slabs),
            N.int_array(out_sizes), N.int_array(col_offsets), S, r_max, N.ptr(_i32(rank_per_slot, "rank_per_slot")),
            N.ptr(scale_per_slot), N.ptr(_i32(tts, "token_to_slot")), N.ptr(_i32(srt, "sorted")), N.ptr(_i32(ids, "slot ids")),
            N.ptr(_i32(cnt, "counts")), N.ptr(_i32(off, "offsets")), n_buckets, float(scaling), N.dtype_code(x.dtype),
            tmp_ptr, peers, rank, tp, capacity, N.current_stream(x.device)))
