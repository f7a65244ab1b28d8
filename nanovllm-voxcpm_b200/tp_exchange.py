"""Peer-memory exchange of the row-parallel LoRA intermediate (tensor parallelism).

``TpExchange`` owns one symmetric buffer per rank (``torch.distributed._symmetric_memory``: the same
allocation mapped into every rank of the group, peers reachable over NVLink) and sums fp32 partials
over the tensor-parallel group with ``lora_b200_tp_allreduce``: one kernel per exchange, no library
collective. It serves ``LoRARowParallelLinear`` in ``lora_tp_mode="peer_exchange"``, where each rank
shrinks on its input shard, the ``[n, T, r]`` partials are summed here, and each rank expands only
its ``out / tp`` columns of ``lora_B``; the base output's own ``[T, out]`` all-reduce
(``nanovllm_voxcpm/layers/lora.py:722-742``) then assembles the full delta exactly once.

Every rank must call :meth:`all_reduce_` in the same order. Multicast is not used (plain peer stores).
"""

from __future__ import annotations

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
        self._peers = (N.c_void_p * self.tp)(*[int(p) for p in self._handle.buffer_ptrs])
        dist.barrier(self.group)  # every rank's buffer is zeroed and mapped before the first push

    def all_reduce_(self, partial: torch.Tensor) -> torch.Tensor:
        """In place: ``partial`` (fp32, contiguous, numel % 4 == 0) becomes the sum over the group."""
        N.require_cuda(partial)
        if partial.dtype != torch.float32 or not partial.is_contiguous():
            raise ValueError("the exchanged partial must be a contiguous float32 tensor")
        with torch.cuda.device(partial.device):
            N.check(N.lib().lora_b200_tp_allreduce(partial.data_ptr(), partial.data_ptr(), partial.numel(), self._peers,
                                                   self.rank, self.tp, self.capacity, N.current_stream(partial.device)))
        return partial
