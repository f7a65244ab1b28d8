"""Per-domain LoRA step context (mirror of ``nanovllm_voxcpm/utils/context.py:21-35,73-155``).

The runner publishes one ``LoRAContext`` per domain and step; every LoRA layer of
that domain reads it.  Contexts are process-global by design (one runner per process).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

LM_LORA_DOMAIN = "lm_domain"
PROJ_LORA_DOMAIN = "proj_domain"
DIT_LORA_DOMAIN = "dit_domain"


@dataclass
class LoRAContext:
    token_to_slot: torch.Tensor | None = None
    token_indices_sorted_by_slot: torch.Tensor | None = None
    active_slot_ids: torch.Tensor | None = None
    num_tokens_per_slot: torch.Tensor | None = None
    slot_start_offsets: torch.Tensor | None = None
    no_lora_flag: bool = True
    num_active_loras: int = 0
    #: Row ranges of a step that mixes batch kinds, e.g. single-token decode rows next to a prefill chunk:
    #: ``[(first_row, end_row, LoRAContext of those rows), ...]``. The layers then issue one multi-LoRA call per
    #: range (the decode kernel for the scattered rows, the tensor-core kernels for the request-contiguous ones)
    #: instead of one call that suits neither. The reference's scheduler never mixes the two kinds
    #: (``nanovllm_voxcpm/engine/scheduler.py:108-140``), so its contexts have no such field.
    parts: list | None = None
    # LoRAMetadata view shared by all layers of the domain within one step
    _cached_metadata: object | None = field(default=None, repr=False, compare=False)


_DOMAINS: dict[str, LoRAContext] = {}


def get_lora_context(domain: str = LM_LORA_DOMAIN) -> LoRAContext:
    return _DOMAINS.get(domain) or LoRAContext()


def set_lora_context(lora_context: LoRAContext, *, domain: str = LM_LORA_DOMAIN) -> None:
    lora_context._cached_metadata = None
    _DOMAINS[domain] = lora_context


def reset_lora_context(domain: str | None = None) -> None:
    if domain is None:
        _DOMAINS.clear()
    else:
        _DOMAINS.pop(domain, None)


def build_lora_context_from_token_to_slot(token_to_slot: torch.Tensor | None) -> LoRAContext:
    """Eager-plan metadata from a device (or CPU) slot map: only slots >= 0 get a
    bucket, ascending slot id, original token order inside a bucket
    (``utils/context.py:77-116``)."""
    if token_to_slot is None or token_to_slot.numel() == 0:
        return LoRAContext(token_to_slot=token_to_slot, no_lora_flag=True, num_active_loras=0)
    tts = token_to_slot.to(dtype=torch.int32)
    keep = tts >= 0
    if not bool(keep.any()):
        return LoRAContext(token_to_slot=tts, no_lora_flag=True, num_active_loras=0)
    rows = torch.nonzero(keep, as_tuple=False).flatten()
    order = torch.sort(tts[rows], stable=True).indices
    active, counts = torch.unique(tts[rows], sorted=True, return_counts=True)
    offsets = torch.zeros(active.numel() + 1, dtype=torch.int32, device=tts.device)
    offsets[1:] = torch.cumsum(counts, dim=0)
    return LoRAContext(
        token_to_slot=tts,
        token_indices_sorted_by_slot=rows[order].to(torch.int32),
        active_slot_ids=active.to(torch.int32),
        num_tokens_per_slot=counts.to(torch.int32),
        slot_start_offsets=offsets,
        no_lora_flag=False,
        num_active_loras=int(active.numel()),
    )


def build_mixed_lora_context(token_to_slot: torch.Tensor, split_rows: list[int]) -> LoRAContext:
    """Context of a step whose rows ``[0, split_rows[0])``, ``[split_rows[0], split_rows[1])``, ... are batches of
    different kinds (decode rows first, then prefill chunks): every range gets its own eager-plan metadata."""
    tts = token_to_slot.to(dtype=torch.int32)
    bounds = [0, *[int(r) for r in split_rows], int(tts.numel())]
    parts = []
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        if hi > lo:
            parts.append((lo, hi, build_lora_context_from_token_to_slot(tts[lo:hi])))
    whole = LoRAContext(token_to_slot=tts, no_lora_flag=all(p[2].no_lora_flag for p in parts),
                        num_active_loras=max([p[2].num_active_loras for p in parts], default=0))
    whole.parts = parts
    return whole


def set_lora_context_from_token_to_slot(token_to_slot: torch.Tensor | None, *, domain: str = LM_LORA_DOMAIN) -> None:
    set_lora_context(build_lora_context_from_token_to_slot(token_to_slot), domain=domain)
