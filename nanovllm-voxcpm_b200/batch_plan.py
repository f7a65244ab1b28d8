"""Host-side batch metadata of a step: token->slot list -> bucket arrays -> device context.

Mirrors the metadata half of ``nanovllm_voxcpm/engine/lora_manager.py:68-180`` (batch
plan, one pinned H2D copy) and the fixed-capacity CUDA-graph buffers of
``nanovllm_voxcpm/engine/model_runner.py:718-817``.  The arrays produced here are the
index inputs of the kernels, so their layout is kept value-for-value.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from .context import LoRAContext


@dataclass
class LoRABatchPlan:
    adapter_to_slot: dict[int, int]
    token_to_slot: list[int]
    token_indices_sorted_by_slot: list[int]
    active_slot_ids: list[int]
    num_tokens_per_slot: list[int]
    slot_start_offsets: list[int]


def bucket_arrays(token_to_slot) -> tuple[list[int], list[int], list[int], list[int]]:
    """(sorted token rows, active slot ids, counts, exclusive offsets) of an eager plan.

    Stable counting sort: ascending slot id, original order inside a slot, rows with
    slot < 0 left out (``engine/lora_manager.py:77-91``)."""
    tts = np.asarray(token_to_slot, dtype=np.int64).reshape(-1)
    rows = np.nonzero(tts >= 0)[0]
    if rows.size == 0:
        return [], [], [], [0]
    order = np.argsort(tts[rows], kind="stable")
    active, counts = np.unique(tts[rows], return_counts=True)
    offsets = np.concatenate([[0], np.cumsum(counts)])
    return rows[order].tolist(), active.tolist(), counts.tolist(), offsets.tolist()


def build_lora_batch_plan_from_token_to_slot(adapter_to_slot: dict[int, int], token_to_slot: list[int]) -> LoRABatchPlan:
    srt, active, counts, offsets = bucket_arrays(token_to_slot)
    return LoRABatchPlan(adapter_to_slot, list(token_to_slot), srt, active, counts, offsets)


def expand_token_counts(slots_per_seq: list[int], token_counts: list[int]) -> list[int]:
    """Per-sequence slot -> per-token slot (``engine/lora_manager.py:371-404``)."""
    out: list[int] = []
    for slot, count in zip(slots_per_seq, token_counts):
        out.extend([slot] * count)
    return out


def _to_device_packed(lists: list[list[int]], device) -> list[torch.Tensor]:
    """All int lists in ONE pinned buffer and one H2D copy; views are returned
    (``engine/lora_manager.py:118-146``)."""
    sizes = [len(x) for x in lists]
    total = sum(sizes)
    if total == 0:
        return [torch.empty(0, dtype=torch.int32, device=device) for _ in lists]
    flat = np.concatenate([np.asarray(x, dtype=np.int32) for x in lists if len(x)])
    host = torch.from_numpy(flat)
    dev = torch.device(device)
    if dev.type == "cuda":
        host = host.pin_memory()
    packed = host.to(dev, non_blocking=True)
    views, pos = [], 0
    for s in sizes:
        views.append(packed[pos : pos + s])
        pos += s
    return views


def build_lora_context_from_batch_plan(plan: LoRABatchPlan, device="cuda") -> LoRAContext:
    if not plan.active_slot_ids:
        (tts,) = _to_device_packed([plan.token_to_slot], device)
        return LoRAContext(token_to_slot=tts, no_lora_flag=True, num_active_loras=0)
    tts, srt, ids, cnt, off = _to_device_packed(
        [plan.token_to_slot, plan.token_indices_sorted_by_slot, plan.active_slot_ids, plan.num_tokens_per_slot,
         plan.slot_start_offsets],
        device,
    )
    return LoRAContext(tts, srt, ids, cnt, off, no_lora_flag=False, num_active_loras=len(plan.active_slot_ids))


def build_lora_context_from_slot_list(token_to_slot: list[int], device="cuda") -> LoRAContext:
    return build_lora_context_from_batch_plan(build_lora_batch_plan_from_token_to_slot({}, token_to_slot), device)


@dataclass
class GraphLoRABuffers:
    """Fixed-capacity metadata of one domain for CUDA-graph replay.

    ``max_loras + 1`` buckets whose ids are ``[-1, 0, 1, ...]``: bucket 0 is the
    "no adapter" id and always holds 0 tokens, the tokens of slot ``s`` sit in bucket
    ``s + 1``; the tail of the sorted-index buffer keeps stale values that no kernel
    reads (``engine/model_runner.py:718-725,774-797``)."""

    token_to_slot: torch.Tensor
    token_indices_sorted_by_slot: torch.Tensor
    active_slot_ids: torch.Tensor
    num_tokens_per_slot: torch.Tensor
    slot_start_offsets: torch.Tensor
    _staging: torch.Tensor | None = field(default=None, repr=False)

    @staticmethod
    def make(max_rows: int, max_loras: int, device="cuda") -> "GraphLoRABuffers":
        buckets = max_loras + 1
        i32 = dict(dtype=torch.int32, device=device)
        return GraphLoRABuffers(
            token_to_slot=torch.full((max_rows,), -1, **i32),
            token_indices_sorted_by_slot=torch.arange(max_rows, **i32),
            active_slot_ids=torch.arange(-1, buckets - 1, **i32),
            num_tokens_per_slot=torch.zeros(buckets, **i32),
            slot_start_offsets=torch.zeros(buckets + 1, **i32),
        )

    @property
    def num_buckets(self) -> int:
        return self.active_slot_ids.numel()

    def load_plan(self, plan: LoRABatchPlan) -> None:
        """Write one step's plan into the graph buffers (values as in
        ``_copy_lora_domain_to_graph_vars``): slot map prefix then -1, sorted-index
        prefix, counts scattered to ``slot + 1``, offsets = running sum."""
        rows = self.token_to_slot.numel()
        buckets = self.num_buckets
        n = len(plan.token_to_slot)
        if n > rows:
            raise ValueError(f"plan has {n} rows, graph buffers hold {rows}")
        tts = np.full(rows, -1, dtype=np.int32)
        tts[:n] = plan.token_to_slot
        counts = np.zeros(buckets, dtype=np.int32)
        for slot, c in zip(plan.active_slot_ids, plan.num_tokens_per_slot):
            if slot + 1 >= buckets:
                raise ValueError(f"slot {slot} outside the {buckets - 1} graph slots")
            counts[slot + 1] = c
        offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        srt = np.asarray(plan.token_indices_sorted_by_slot, dtype=np.int32)
        views = _to_device_packed([tts.tolist(), srt.tolist(), counts.tolist(), offsets.tolist()], self.token_to_slot.device)
        self.token_to_slot.copy_(views[0], non_blocking=True)
        if srt.size:
            self.token_indices_sorted_by_slot[: srt.size].copy_(views[1], non_blocking=True)
        self.num_tokens_per_slot.copy_(views[2], non_blocking=True)
        self.slot_start_offsets.copy_(views[3], non_blocking=True)

    def load_token_to_slot_on_device(self, token_to_slot: torch.Tensor) -> None:
        """Same buffers as :meth:`load_plan`, built on the GPU from a device-resident slot map in two
        launches (a copy and ``lora_b200_build_metadata``): no Python loop over the rows, no staging
        copy, nothing to synchronise. Slot ids outside the graph slots count as "no adapter"."""
        from . import _native as N

        n = token_to_slot.numel()
        rows = self.token_to_slot.numel()
        if n > rows:
            raise ValueError(f"slot map has {n} rows, graph buffers hold {rows}")
        self.token_to_slot[:n].copy_(token_to_slot, non_blocking=True)
        if n < rows:
            self.token_to_slot[n:].fill_(-1)
        N.build_metadata(self.token_to_slot, self.num_buckets - 1, N.META_GRAPH, self.token_indices_sorted_by_slot,
                         None, self.num_tokens_per_slot, self.slot_start_offsets)

    def context(self, token_count: int, no_lora_flag: bool = False) -> LoRAContext:
        return LoRAContext(
            token_to_slot=self.token_to_slot[:token_count],
            token_indices_sorted_by_slot=self.token_indices_sorted_by_slot[:token_count],
            active_slot_ids=self.active_slot_ids,
            num_tokens_per_slot=self.num_tokens_per_slot,
            slot_start_offsets=self.slot_start_offsets,
            no_lora_flag=no_lora_flag,
            num_active_loras=self.num_buckets,
        )
