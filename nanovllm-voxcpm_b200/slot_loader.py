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
arena, which is copied to the device in one piece without being repacked on the host.
"""

from __future__ import annotations

import ctypes

import torch
import torch.nn as nn

from . import _native as N
from . import layers as L


class _Desc(ctypes.Structure):
    _fields_ = [
        ("dst", ctypes.c_uint64), ("src_offset", ctypes.c_int64), ("kind", ctypes.c_int32),
        ("dst_rows", ctypes.c_int32), ("dst_cols", ctypes.c_int32), ("src_rows", ctypes.c_int32),
        ("src_cols", ctypes.c_int32), ("src_ld", ctypes.c_int32), ("src_dtype", ctypes.c_int32),
        ("dst_dtype", ctypes.c_int32), ("scale", ctypes.c_float), ("ivalue", ctypes.c_int32),
        ("pad0", ctypes.c_int32), ("pad1", ctypes.c_int32),
    ]


assert ctypes.sizeof(_Desc) == 64


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

    # ------------------------------------------------------------------ staging
    def _buffers(self, nbytes: int) -> tuple[torch.Tensor, torch.Tensor]:
        if self._host is None or self._host.numel() < nbytes:
            cap = max(nbytes, 1 << 20)
            self._host = torch.empty(cap, dtype=torch.uint8).pin_memory()
            self._dev = torch.empty(cap, dtype=torch.uint8, device=self.device)
        return self._host, self._dev

    @staticmethod
    def _parts(module, lora_a, lora_b):
        """Per-slice (A payload, B payload) of a module, in ``_a_slices()`` / ``_b_slices()`` order."""
        if isinstance(lora_b, list):
            return list(lora_a), list(lora_b)
        return [lora_a], [lora_b]

    # ------------------------------------------------------------------ load
    def load_slot(self, slot_id: int, payload) -> None:
        arena = None
        if hasattr(payload, "modules"):  # a LoRAModelPayload (adapter_checkpoint / the reference's dataclass)
            arena = getattr(payload, "arena", None)
            payload = {name: (m.lora_a, m.lora_b, m.effective_rank, m.scaling) for name, m in payload.modules.items()}
        if arena is not None and (arena.device.type != "cpu" or arena.dtype != torch.uint8 or not arena.is_contiguous()):
            arena = None
        arena_lo = arena.data_ptr() if arena is not None else 0
        arena_hi = arena_lo + (arena.numel() if arena is not None else 0)
        descs: list[_Desc] = []
        in_arena: list[_Desc] = []                   # descriptors whose payload is read from the arena's copy
        blobs: list[tuple[int, torch.Tensor]] = []   # (byte offset, host tensor) of every other payload tensor
        cursor = 0
        max_elems = 1

        def region(dst: torch.Tensor, src: torch.Tensor | None, rows_used: int, cols_used: int, scale: float):
            nonlocal cursor, max_elems
            d = _Desc()
            d.dst, d.kind = dst.data_ptr(), 0
            d.dst_rows, d.dst_cols = dst.shape
            d.dst_dtype = N.dtype_code(dst.dtype)
            d.scale = scale
            if src is None:
                d.src_rows = d.src_cols = d.src_ld = 0
                d.src_dtype, d.src_offset = N.dtype_code(torch.float32), 0
            elif (arena is not None and src.device.type == "cpu" and src.dim() == 2 and src.stride(1) == 1
                  and arena_lo <= src.data_ptr() and src.data_ptr() + src.element_size() * (
                      (src.size(0) - 1) * src.stride(0) + src.size(1)) <= arena_hi):
                # a view of the payload's arena: the arena is copied as it lies, nothing is repacked
                d.src_rows, d.src_cols, d.src_ld = rows_used, cols_used, src.stride(0)
                d.src_dtype, d.src_offset = N.dtype_code(src.dtype), src.data_ptr() - arena_lo
                in_arena.append(d)
            else:
                src = src.detach()
                if src.device.type != "cpu":
                    src = src.cpu()
                src = src.contiguous()
                d.src_rows, d.src_cols, d.src_ld = rows_used, cols_used, src.size(1)
                d.src_dtype, d.src_offset = N.dtype_code(src.dtype), cursor  # offset patched after the table is sized
                blobs.append((cursor, src))
                cursor += (src.numel() * src.element_size() + 15) & ~15
            max_elems = max(max_elems, dst.numel())
            descs.append(d)

        def scalar(dst: torch.Tensor, value):
            d = _Desc()
            d.dst = dst.data_ptr()
            if dst.dtype == torch.int32:
                d.kind, d.ivalue = 1, int(value)
            else:
                d.kind, d.scale, d.dst_dtype = 2, float(value), N.dtype_code(dst.dtype)
            descs.append(d)

        def record(module, rank: int, scaling: float):
            scalar(module.effective_lora_rank[slot_id], rank)
            scalar(module.lora_scaling[slot_id], scaling)
            scalar(module.lora_base_scaling[slot_id], scaling)

        for name, (lora_a, lora_b, rank, scaling) in payload.items():
            if name not in self.modules:
                raise ValueError(f"Unknown LoRA target module '{name}'")
            self.modules[name].validate_slot_lora_payload(lora_a, lora_b, rank, scaling)
        if not 0 <= slot_id < next(iter(self.modules.values())).max_loras:
            raise ValueError(f"slot {slot_id} outside the resident slots")
        # what the previous occupant had and the new adapter does not cover is cleared
        for name in self._loaded.get(slot_id, []):
            if name not in payload:
                module = self.modules[name]
                for slab in (*module._a_slices(), *module._b_slices()):
                    region(slab[slot_id], None, 0, 0, 0.0)
                record(module, 0, 0.0)
        for name, (lora_a, lora_b, rank, scaling) in payload.items():
            module = self.modules[name]
            a_parts, b_parts = self._parts(module, lora_a, lora_b)
            for slab, part in zip(module._a_slices(), a_parts):
                region(slab[slot_id], part, rank, part.size(1), 1.0)
            for slab, part in zip(module._b_slices(), b_parts):
                region(slab[slot_id], part, part.size(0), rank, float(scaling))
            record(module, rank, scaling)

        table_bytes = len(descs) * 64
        if self._copied is not None:
            self._copied.synchronize()  # the previous admission's copy still reads the pinned buffer until then
        # device layout: [descriptor table | repacked payload tensors | the arena as it lies on the host]
        arena_base = (table_bytes + cursor + 63) & ~63
        arena_bytes = arena.numel() if in_arena else 0
        host, dev = self._buffers(arena_base + arena_bytes)
        from_arena = {id(d) for d in in_arena}
        for d in descs:
            if d.kind == 0 and d.src_rows > 0:
                d.src_offset += arena_base if id(d) in from_arena else table_bytes
        table = (_Desc * len(descs))(*descs)
        host[:table_bytes].copy_(torch.frombuffer(bytearray(bytes(table)), dtype=torch.uint8))
        for off, src in blobs:
            n = src.numel() * src.element_size()
            host[table_bytes + off: table_bytes + off + n].copy_(src.view(torch.uint8).reshape(-1))
        total = table_bytes + cursor
        with torch.cuda.device(self.device):
            dev[:total].copy_(host[:total], non_blocking=True)
            if arena_bytes:
                # asynchronous when the arena is pinned; the payload must stay unchanged until the copy has run
                dev[arena_base: arena_base + arena_bytes].copy_(arena, non_blocking=True)
            self._copied = torch.cuda.Event()
            self._copied.record()
            N.check(N.lib().lora_b200_load_slot(dev.data_ptr(), len(descs), max_elems, N.current_stream(self.device)))
        # host mirrors of the layers (the kernel wrote the device buffers)
        for name in self._loaded.get(slot_id, []):
            if name not in payload:
                self._mirror(self.modules[name], slot_id, 0, 0.0)
        for name, (_, _, rank, scaling) in payload.items():
            self._mirror(self.modules[name], slot_id, rank, scaling)
        self._loaded[slot_id] = list(payload.keys())

    @staticmethod
    def _mirror(module, slot_id: int, rank: int, scaling: float) -> None:
        module._effective_lora_rank_values[slot_id] = rank
        module._lora_scaling_values[slot_id] = scaling
        module._lora_base_scaling_values[slot_id] = scaling
