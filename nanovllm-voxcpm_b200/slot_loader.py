"""Adapter admission: all slabs of one slot written by one copy and one kernel.

``SlotLoader.load_slot(slot_id, payload)`` does what the reference's ``_load_lora_slot`` does module by
module (``nanovllm_voxcpm/engine/model_runner.py:389-420``: clear what the slot's previous occupant
had loaded, then ``set_slot_lora`` per module, i.e. zero the slot, copy the first ``effective_rank`` rows /
columns, fold the scaling into B, record rank and scaling - ``layers/lora.py:395-417``) with ONE packed
pinned staging buffer, one host->device copy and one launch of ``lora_b200_load_slot``. The slabs and
the per-slot buffers end up bit-identical to the module-by-module path; the layers' own validators and
host mirrors are used unchanged.

``payload`` maps module names to ``(lora_a, lora_b, effective_rank, scaling)`` in the form each
layer's ``set_slot_lora`` takes (multi-slice layers: ``lora_a [slices, rank, in]`` and a list of
``lora_b``); tensors may live on the host (the usual case) or on the device. A ``LoRAModelPayload``
(``adapter_checkpoint.load_lora_checkpoint``) is taken as it is; its tensors are views of one pinned
arena, which is copied to the device in one piece without being repacked on the host, and the
descriptor table of such a payload is planned once and re-aimed at the slot on later admissions.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.nn as nn

from . import _native as N
from . import layers as L

# layout of SlotLoadDesc in csrc/slot_loader.cuh
_DESC = np.dtype([("dst", "<u8"), ("src_offset", "<i8"), ("kind", "<i4"), ("dst_rows", "<i4"), ("dst_cols", "<i4"),
                  ("src_rows", "<i4"), ("src_cols", "<i4"), ("src_ld", "<i4"), ("src_dtype", "<i4"),
                  ("dst_dtype", "<i4"), ("scale", "<f4"), ("ivalue", "<i4"), ("pad0", "<i4"), ("pad1", "<i4")])
assert _DESC.itemsize == 64
_KIND_REGION, _KIND_INT, _KIND_FLOAT = 0, 1, 2
_SRC_NONE, _SRC_BLOB, _SRC_ARENA = 0, 1, 2
_PLAN_CACHE_ENTRIES = 256


@dataclass
class _Plan:
    """Descriptor table of one payload, aimed at slot 0; ``dst + slot * slot_stride`` aims it elsewhere."""

    payload: object                 # the LoRAModelPayload this was planned for (None: not cached)
    cleared: tuple[str, ...]        # modules of the previous occupant that this plan zeroes
    table: np.ndarray               # _DESC records, src_offset relative to the blob area / the arena
    slot_stride: np.ndarray         # bytes from a slot's destination to the next slot's, per record
    src_kind: np.ndarray            # _SRC_* per record
    blobs: list                     # (byte offset in the blob area, contiguous host tensor)
    blob_bytes: int
    arena: torch.Tensor | None      # copied as it lies when any record reads from it
    max_elems: int
    mirrors: list                   # (module, rank, scaling) for the layers' host-side lists
    names: list[str]
    guard: int                      # address of the first slab when the plan was made


class SlotLoader:
    def __init__(self, model: nn.Module):
        self.modules = {name: m for name, m in model.named_modules()
                        if isinstance(m, L._LORA_LAYER_TYPES) and m.lora_enabled}
        if not self.modules:
            raise ValueError("the model has no LoRA-enabled module")
        self.device = next(iter(self.modules.values())).weight.device
        self._loaded: dict[int, list[str]] = {}   # slot -> modules its occupant populated
        self._host: torch.Tensor | None = None    # pinned staging (grow-only)
        self._dev: torch.Tensor | None = None
        self._copied: torch.cuda.Event | None = None  # the staging buffer is free again once this has passed
        self._plans: dict[tuple[int, tuple[str, ...]], _Plan] = {}

    # ------------------------------------------------------------------ staging
    def _buffers(self, nbytes: int) -> tuple[torch.Tensor, torch.Tensor]:
        if self._host is None or self._host.numel() < nbytes:
            cap = max(nbytes, 1 << 20)
            self._host = torch.empty(cap, dtype=torch.uint8).pin_memory()
            self._dev = torch.empty(cap, dtype=torch.uint8, device=self.device)
        return self._host, self._dev

    def _guard(self) -> int:
        return next(iter(self.modules.values()))._a_slices()[0].data_ptr()

    def forget(self, payload) -> None:
        """Drops the cached plans of ``payload`` (and with them the references that keep its arena alive)."""
        for key in [k for k, p in self._plans.items() if p.payload is payload]:
            del self._plans[key]

    # ------------------------------------------------------------------ plan
    def _plan(self, payload_obj, payload: dict, arena, cleared: tuple[str, ...]) -> _Plan:
        if arena is not None and (arena.device.type != "cpu" or arena.dtype != torch.uint8 or not arena.is_contiguous()):
            arena = None
        arena_lo = arena.data_ptr() if arena is not None else 0
        arena_hi = arena_lo + (arena.numel() if arena is not None else 0)
        rows: list[tuple] = []
        strides: list[int] = []
        kinds: list[int] = []
        blobs: list[tuple[int, torch.Tensor]] = []
        cursor = 0
        max_elems = 1
        f32 = N.dtype_code(torch.float32)

        def region(slab: torch.Tensor, src: torch.Tensor | None, rows_used: int, cols_used: int, scale: float):
            nonlocal cursor, max_elems
            _, dst_rows, dst_cols = slab.shape
            dst_dtype = N.dtype_code(slab.dtype)
            if src is None:
                rec, kind = (0, 0, 0, f32, 0), _SRC_NONE
            elif (arena is not None and src.device.type == "cpu" and src.dim() == 2 and src.stride(1) == 1
                  and arena_lo <= src.data_ptr() and src.data_ptr() + src.element_size() * (
                      (src.size(0) - 1) * src.stride(0) + src.size(1)) <= arena_hi):
                # a view of the payload's arena: the arena is copied as it lies, nothing is repacked
                rec, kind = (rows_used, cols_used, src.stride(0), N.dtype_code(src.dtype), src.data_ptr() - arena_lo), _SRC_ARENA
            else:
                src = src.detach()
                if src.device.type != "cpu":
                    src = src.cpu()
                src = src.contiguous()
                rec, kind = (rows_used, cols_used, src.size(1), N.dtype_code(src.dtype), cursor), _SRC_BLOB
                blobs.append((cursor, src))
                cursor += (src.numel() * src.element_size() + 15) & ~15
            max_elems = max(max_elems, dst_rows * dst_cols)
            rows.append((slab.data_ptr(), rec[4], _KIND_REGION, dst_rows, dst_cols, rec[0], rec[1], rec[2], rec[3],
                         dst_dtype, scale, 0, 0, 0))
            strides.append(slab.stride(0) * slab.element_size())
            kinds.append(kind)

        def scalar(buf: torch.Tensor, value):
            if buf.dtype == torch.int32:
                rows.append((buf.data_ptr(), 0, _KIND_INT, 0, 0, 0, 0, 0, 0, 0, 0.0, int(value), 0, 0))
            else:
                rows.append((buf.data_ptr(), 0, _KIND_FLOAT, 0, 0, 0, 0, 0, 0, N.dtype_code(buf.dtype), float(value), 0, 0, 0))
            strides.append(buf.stride(0) * buf.element_size())
            kinds.append(_SRC_NONE)

        def record(module, rank: int, scaling: float):
            scalar(module.effective_lora_rank, rank)
            scalar(module.lora_scaling, scaling)
            scalar(module.lora_base_scaling, scaling)

        mirrors = []
        # what the previous occupant had and the new adapter does not cover is cleared
        for name in cleared:
            module = self.modules[name]
            for slab in (*module._a_slices(), *module._b_slices()):
                region(slab, None, 0, 0, 0.0)
            record(module, 0, 0.0)
            mirrors.append((module, 0, 0.0))
        for name, (lora_a, lora_b, rank, scaling) in payload.items():
            module = self.modules[name]
            a_parts, b_parts = (list(lora_a), list(lora_b)) if isinstance(lora_b, list) else ([lora_a], [lora_b])
            for slab, part in zip(module._a_slices(), a_parts):
                region(slab, part, rank, part.size(1), 1.0)
            for slab, part in zip(module._b_slices(), b_parts):
                region(slab, part, part.size(0), rank, float(scaling))
            record(module, rank, scaling)
            mirrors.append((module, rank, scaling))
        kinds_np = np.asarray(kinds, dtype=np.int8)
        return _Plan(payload=payload_obj, cleared=cleared, table=np.array(rows, dtype=_DESC),
                     slot_stride=np.asarray(strides, dtype=np.uint64), src_kind=kinds_np, blobs=blobs, blob_bytes=cursor,
                     arena=arena if bool((kinds_np == _SRC_ARENA).any()) else None, max_elems=max_elems, mirrors=mirrors,
                     names=list(payload.keys()), guard=self._guard())

    # ------------------------------------------------------------------ load
    def load_slot(self, slot_id: int, payload) -> None:
        payload_obj = payload if hasattr(payload, "modules") else None  # a LoRAModelPayload
        if not 0 <= slot_id < next(iter(self.modules.values())).max_loras:
            raise ValueError(f"slot {slot_id} outside the resident slots")
        names = payload_obj.modules.keys() if payload_obj is not None else payload.keys()
        cleared = tuple(n for n in self._loaded.get(slot_id, []) if n not in names)
        plan = self._plans.get((id(payload_obj), cleared)) if payload_obj is not None else None
        if plan is not None and (plan.payload is not payload_obj or plan.guard != self._guard()):
            plan = None
        if plan is None:
            arena = getattr(payload_obj, "arena", None)
            if payload_obj is not None:
                payload = {n: (m.lora_a, m.lora_b, m.effective_rank, m.scaling) for n, m in payload_obj.modules.items()}
            for name, (lora_a, lora_b, rank, scaling) in payload.items():
                if name not in self.modules:
                    raise ValueError(f"Unknown LoRA target module '{name}'")
                self.modules[name].validate_slot_lora_payload(lora_a, lora_b, rank, scaling)
            plan = self._plan(payload_obj, payload, arena, cleared)
            if payload_obj is not None and not plan.blobs:
                if len(self._plans) >= _PLAN_CACHE_ENTRIES:
                    del self._plans[next(iter(self._plans))]
                self._plans[(id(payload_obj), cleared)] = plan

        n_desc = len(plan.table)
        table_bytes = n_desc * 64
        # device layout: [descriptor table | repacked payload tensors | the arena as it lies on the host]
        arena_base = (table_bytes + plan.blob_bytes + 63) & ~63
        arena_bytes = plan.arena.numel() if plan.arena is not None else 0
        table = plan.table.copy()
        table["dst"] += plan.slot_stride * np.uint64(slot_id)
        table["src_offset"] += np.where(plan.src_kind == _SRC_ARENA, arena_base,
                                        np.where(plan.src_kind == _SRC_BLOB, table_bytes, 0)).astype(np.int64)
        if self._copied is not None:
            self._copied.synchronize()  # the previous admission's copy still reads the pinned buffer until then
        host, dev = self._buffers(arena_base + arena_bytes)
        host[:table_bytes].copy_(torch.from_numpy(table.view(np.uint8).reshape(-1)))
        for off, src in plan.blobs:
            n = src.numel() * src.element_size()
            host[table_bytes + off: table_bytes + off + n].copy_(src.view(torch.uint8).reshape(-1))
        total = table_bytes + plan.blob_bytes
        with N.on_device(self.device):
            dev[:total].copy_(host[:total], non_blocking=True)
            if arena_bytes:
                # asynchronous when the arena is pinned; the payload must stay unchanged until the copy has run
                dev[arena_base: arena_base + arena_bytes].copy_(plan.arena, non_blocking=True)
            self._copied = torch.cuda.Event()
            self._copied.record()
            N.check(N.lib().lora_b200_load_slot(dev.data_ptr(), n_desc, plan.max_elems, N.current_stream(self.device)))
        # host mirrors of the layers (the kernel wrote the device buffers)
        for module, rank, scaling in plan.mirrors:
            module._effective_lora_rank_values[slot_id] = rank
            module._lora_scaling_values[slot_id] = scaling
            module._lora_base_scaling_values[slot_id] = scaling
        self._loaded[slot_id] = list(plan.names)
