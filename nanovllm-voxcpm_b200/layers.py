"""LoRA linear layers of the LM backbone (qkv / o / gate_up / down), B200 path.

Same constructors, slab attribute names (``lora_A``, ``lora_B_q|k|v``, ``lora_B_<i>``,
``lora_B``, ``effective_lora_rank``, ``lora_scaling``, ``lora_base_scaling``), slot
loading API (``set_slot_lora`` / ``clear_slot_lora`` / ``validate_slot_lora_payload`` /
``reset_lora_parameters``) and forward semantics as the reference's
``nanovllm_voxcpm/layers/lora.py`` (``LoRAQKVParallelLinear`` :244-465,
``LoRAMergedColumnParallelLinear`` :468-667, ``LoRARowParallelLinear`` :670-797,
``LoRALinear`` :800-904), so a runner's slot loader and ``iter_lora_modules`` keep
working.  Differences are internal: every forward issues one fused launch that writes
the LoRA delta in place at the slice's column offset (also for partial target sets, so
there is no split / cat round trip), and the per-slot effective rank is handed to the
kernel so zero padding of mixed-rank slabs is not multiplied.

Slab invariants the kernels rely on (kept by ``set_slot_lora``): a slot is zeroed before
it is written, only the first ``effective_rank`` rows / columns are filled, and the
adapter's scaling is folded into ``lora_B`` (``layers/lora.py:404-417``).
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .context import LM_LORA_DOMAIN, get_lora_context, set_lora_context
from .distributed import get_tp_rank, get_tp_world_size
from .lora import B200LoRABackend, LoRAMetadata, get_backend


#: opt-in: route large bf16 batches through the fused base-GEMM + LoRA tensor-core kernel
FUSED_LINEAR = False
#: True: bf16 batches of a layer without bias compute the LoRA delta FIRST (``lora_b200_delta`` into the output
#: buffer, -0.0 in rows without adapter) and let the base GEMM accumulate into it (``addmm_``): in decode the
#: multi-LoRA launch no longer waits for the GEMM and overlaps the kernel before it, in prefill the delta tiles are
#: stored instead of being reduce-added into y
LORA_FIRST = False


def _get_world_size() -> int:
    return get_tp_world_size()


def _get_rank() -> int:
    return get_tp_rank()


def divide(numerator: int, denominator: int) -> int:
    if numerator % denominator != 0:
        raise ValueError(f"{numerator} is not divisible by {denominator}")
    return numerator // denominator


def _is_cuda_graph_capture() -> bool:
    return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()


class _LoRALayerBase(nn.Module):
    """Slot bookkeeping, context gating and the fused apply shared by the four layers."""

    def __init__(self, max_loras: int, max_lora_rank: int, supports_lora: bool, lora_domain: str = LM_LORA_DOMAIN):
        super().__init__()
        self.max_loras = max_loras
        self.max_lora_rank = max_lora_rank
        self.supports_lora = supports_lora
        self.lora_domain = lora_domain
        self.register_buffer("lora_scaling", torch.zeros(max_loras), persistent=False)
        self.register_buffer("lora_base_scaling", torch.zeros(max_loras), persistent=False)
        self.register_buffer("effective_lora_rank", torch.zeros(max_loras, dtype=torch.int32), persistent=False)
        self._lora_scaling_values = [0.0] * max_loras
        self._lora_base_scaling_values = [0.0] * max_loras
        self._effective_lora_rank_values = [0] * max_loras

    # ------------------------------------------------------------ slab access
    def _a_slices(self) -> list[torch.Tensor]:
        raise NotImplementedError

    def _b_slices(self) -> list[torch.Tensor]:
        raise NotImplementedError

    def _slice_layout(self) -> tuple[list[int], list[int]]:
        """(width, first output column) of every LoRA slice inside the layer output."""
        raise NotImplementedError

    @property
    def lora_enabled(self) -> bool:
        return self.supports_lora

    # --------------------------------------------------------- context gating
    def _resolve_token_slots(self, x_flat: torch.Tensor) -> torch.Tensor | None:
        """The step's slot map, or None when this forward needs no LoRA work
        (``layers/lora.py:78-113``)."""
        if not self.supports_lora:
            return None
        context = get_lora_context(self.lora_domain)
        tts = context.token_to_slot
        if tts is None or context.no_lora_flag or tts.numel() == 0:
            return None
        if tts.device != x_flat.device:
            raise RuntimeError("LoRA token_to_slot must be prepared on the execution device by the model runner")
        if tts.numel() != x_flat.size(0):
            raise RuntimeError(
                "LoRA token_to_slot length does not match flattened input rows: "
                f"token_to_slot={tts.numel()} rows={x_flat.size(0)}"
            )
        # Host-only shortcut: nothing resident in this module. Never taken during graph
        # capture, where the captured launch must stay valid for later slot loads.
        if not _is_cuda_graph_capture() and not any(self._effective_lora_rank_values):
            return None
        return tts

    def _runtime_metadata(self) -> LoRAMetadata | None:
        context = get_lora_context(self.lora_domain)
        if context.token_to_slot is None:
            return None
        meta = context._cached_metadata
        if meta is None:
            meta = LoRAMetadata(
                token_to_slot=context.token_to_slot,
                token_indices_sorted_by_slot=context.token_indices_sorted_by_slot,
                active_slot_ids=context.active_slot_ids,
                num_tokens_per_slot=context.num_tokens_per_slot,
                slot_start_offsets=context.slot_start_offsets,
                no_lora_flag=context.no_lora_flag,
                num_active_loras=context.num_active_loras,
            )
            context._cached_metadata = meta
        return meta  # type: ignore[return-value]

    def _linear(self, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
        """Base linear + LoRA delta of this module.

        Default: cuBLAS (``F.linear``) followed by the fused in-place LoRA add. With
        ``FUSED_LINEAR`` switched on, bf16 batches of at least ``lora.SGMV_MIN_TOKENS`` rows
        take ``lora_b200_linear_lora`` instead: one tensor-core kernel whose accumulator
        receives the delta before the single store of ``y``."""
        mixed = bool(get_lora_context(self.lora_domain).parts)
        if FUSED_LINEAR and not mixed and x.is_cuda and isinstance(get_backend(), B200LoRABackend):
            from .lora import SGMV_MIN_TOKENS, fused_linear_supported, linear_lora

            x_flat = x if x.dim() == 2 else x.reshape(-1, x.size(-1))
            if x_flat.size(0) >= SGMV_MIN_TOKENS and fused_linear_supported(x_flat, weight, self.max_lora_rank):
                token_to_slot = self._resolve_token_slots(x_flat)
                if token_to_slot is not None:
                    widths, cols = self._slice_layout()
                    active = [i for i, w in enumerate(widths) if w > 0]
                    a, b = self._a_slices(), self._b_slices()
                    y = linear_lora(
                        x_flat, weight, bias, [a[i] for i in active], [b[i] for i in active],
                        [widths[i] for i in active], [cols[i] for i in active], token_to_slot, 1.0,
                    )
                    return y if x.dim() == 2 else y.view(*x.shape[:-1], y.size(-1))
        if LORA_FIRST and not mixed and bias is None and x.is_cuda and isinstance(get_backend(), B200LoRABackend):
            from .lora import launch_add

            x_flat = x if x.dim() == 2 else x.reshape(-1, x.size(-1))
            if x_flat.dtype == torch.bfloat16:
                token_to_slot = self._resolve_token_slots(x_flat)
                metadata = self._runtime_metadata()
                widths, cols = self._slice_layout()
                active = [i for i, w in enumerate(widths) if w > 0]
                covered = sorted((cols[i], cols[i] + widths[i]) for i in active)
                whole = bool(covered) and covered[0][0] == 0 and covered[-1][1] == weight.size(0) and all(
                    covered[i][1] == covered[i + 1][0] for i in range(len(covered) - 1))
                if token_to_slot is not None and metadata is not None and whole:
                    # the delta first (its launch does not wait for the GEMM), then the GEMM accumulates into it
                    a, b = self._a_slices(), self._b_slices()
                    y = torch.empty(x_flat.size(0), weight.size(0), dtype=x.dtype, device=x.device)
                    launch_add(y, x_flat, [a[i] for i in active], [b[i] for i in active], [widths[i] for i in active],
                               [cols[i] for i in active], metadata, 1.0, rank_per_slot=self.effective_lora_rank,
                               impl=get_backend().impl, overwrite=True)
                    y.addmm_(x_flat, weight.t())
                    return y if x.dim() == 2 else y.view(*x.shape[:-1], y.size(-1))
        return self._apply_lora(F.linear(x, weight, bias), x)

    def _per_part(self, fn, y: torch.Tensor, x: torch.Tensor) -> torch.Tensor | None:
        """A step that mixes batch kinds (``LoRAContext.parts``): ``fn(y_rows, x_rows)`` once per row range, each
        under that range's own context. Returns None when the step is not mixed."""
        whole = get_lora_context(self.lora_domain)
        if not whole.parts:
            return None
        x_flat = x if x.dim() == 2 else x.reshape(-1, x.size(-1))
        y_flat = y if y.dim() == 2 else y.view(-1, y.size(-1))
        cached = whole._cached_metadata
        try:
            for lo, hi, part in whole.parts:
                meta = part._cached_metadata  # survives the re-publication below: one metadata view per part and step
                set_lora_context(part, domain=self.lora_domain)
                part._cached_metadata = meta
                fn(y_flat[lo:hi], x_flat[lo:hi])
        finally:
            set_lora_context(whole, domain=self.lora_domain)
            whole._cached_metadata = cached
        return y

    def _apply_lora(self, y: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        """Add the LoRA delta of this module to ``y`` in place (fused shrink+expand)."""
        if self._per_part(self._apply_lora, y, x) is not None:
            return y
        x_flat = x if x.dim() == 2 else x.reshape(-1, x.size(-1))
        token_to_slot = self._resolve_token_slots(x_flat)
        if token_to_slot is None:
            return y
        y_flat = y if y.dim() == 2 else y.view(-1, y.size(-1))
        widths, cols = self._slice_layout()
        views = [y_flat[:, c : c + w] for w, c in zip(widths, cols)]
        backend = get_backend()
        metadata = self._runtime_metadata()
        if isinstance(backend, B200LoRABackend):
            # In-place at explicit column offsets; also covers partial target sets.
            from .lora import launch_add

            if metadata is None:
                raise RuntimeError("LoRA metadata must be prepared by the model runner before backend execution")
            active = [i for i, w in enumerate(widths) if w > 0]
            if active:
                a, b = self._a_slices(), self._b_slices()
                launch_add(
                    y_flat, x_flat, [a[i] for i in active], [b[i] for i in active], [widths[i] for i in active],
                    [cols[i] for i in active], metadata, 1.0, rank_per_slot=self.effective_lora_rank,
                    impl=backend.impl,
                )
            return y
        # Foreign backend (e.g. a test double): protocol call, then copy back if it
        # returned fresh tensors (legacy contract of lora.py:283-286).
        contiguous_cover = cols == [sum(widths[:i]) for i in range(len(widths))] and sum(widths) == y_flat.size(1)
        out = backend.add_lora(
            views, x_flat, self._a_slices(), self._b_slices(), indices=token_to_slot, metadata=metadata, scaling=1.0,
            **({"y_packed": y_flat} if contiguous_cover and len(views) > 1 else {}),
        )
        for view, new in zip(views, out):
            if new.data_ptr() != view.data_ptr():
                view.copy_(new)
        return y

    # ------------------------------------------------------------ slot loading
    def _validate_effective_rank(self, effective_rank: int) -> None:
        if effective_rank < 0 or effective_rank > self.max_lora_rank:
            raise ValueError(f"effective_rank={effective_rank} exceeds max_lora_rank={self.max_lora_rank}")

    def _validate_common_slot_payload(self, effective_rank: int, scaling: float) -> None:
        if not self.supports_lora:
            raise ValueError(f"{self.__class__.__name__} does not enable LoRA")
        if effective_rank <= 0:
            raise ValueError(f"effective_rank must be > 0, got {effective_rank}")
        if not math.isfinite(scaling):
            raise ValueError(f"LoRA scaling must be finite, got {scaling}")
        self._validate_effective_rank(effective_rank)

    def _record_slot(self, slot_id: int, effective_rank: int, scaling: float) -> None:
        self.effective_lora_rank[slot_id] = effective_rank
        self.lora_scaling[slot_id] = scaling
        self.lora_base_scaling[slot_id] = scaling
        self._effective_lora_rank_values[slot_id] = effective_rank
        self._lora_scaling_values[slot_id] = scaling
        self._lora_base_scaling_values[slot_id] = scaling

    def _write_slot(self, slot_id: int, a_parts, b_parts, effective_rank: int, scaling: float) -> None:
        """Zero the slot, copy the first ``effective_rank`` rows / columns, fold the
        scaling into B."""
        self._validate_effective_rank(effective_rank)
        r = effective_rank
        with torch.no_grad():
            for slab, part in zip(self._a_slices(), a_parts):
                slab.data[slot_id].zero_()
                slab.data[slot_id, :r].copy_(part[:r])
            for slab, part in zip(self._b_slices(), b_parts):
                slab.data[slot_id].zero_()
                slab.data[slot_id, :, :r].copy_(part[:, :r] * scaling)
        self._record_slot(slot_id, r, scaling)

    def clear_slot_lora(self, slot_id: int) -> None:
        if not self.supports_lora:
            return
        with torch.no_grad():
            for slab in (*self._a_slices(), *self._b_slices()):
                slab.data[slot_id].zero_()
        self._record_slot(slot_id, 0, 0.0)

    def reset_lora_parameters(self) -> None:
        if not self.supports_lora:
            return
        with torch.no_grad():
            for slab in (*self._a_slices(), *self._b_slices()):
                slab.data.zero_()

    def prime_lora_cache(self) -> None:
        """Kept for runner compatibility (``engine/model_runner.py:847-851``); this
        backend has no pointer tables to build before graph capture."""
        backend = get_backend()
        prime = getattr(backend, "prime_slice_caches", None)
        if self.supports_lora and prime is not None:
            prime(self._a_slices(), self._b_slices())

    def set_slot_lora(self, slot_id, lora_a, lora_b, effective_rank, scaling) -> None:
        raise NotImplementedError

    def validate_slot_lora_payload(self, lora_a, lora_b, effective_rank, scaling) -> None:
        raise NotImplementedError


def _check_multi_payload(name, targets, lora_a, lora_b, effective_rank, in_dim, expected_out) -> None:
    if not isinstance(lora_b, list):
        raise ValueError(f"{name} expects lora_b to be a list ordered as layer lora_targets")
    if lora_a.ndim != 3:
        raise ValueError(f"{name} expects 3D lora_a, got shape={tuple(lora_a.shape)}")
    if lora_a.size(0) != len(targets):
        raise ValueError(f"Expected {len(targets)} LoRA A targets, got {lora_a.size(0)}")
    if lora_a.size(1) < effective_rank:
        raise ValueError(f"LoRA A rank dim {lora_a.size(1)} is smaller than effective_rank={effective_rank}")
    if lora_a.size(2) != in_dim:
        raise ValueError(f"Expected lora_a input dim {in_dim}, got {lora_a.size(2)}")
    if len(lora_b) != len(targets):
        raise ValueError(f"Expected {len(targets)} LoRA B tensors ordered as {targets}")
    for target, b in zip(targets, lora_b):
        if b.ndim != 2:
            raise ValueError(f"Target {target!r} expects 2D lora_b, got shape={tuple(b.shape)}")
        if b.size(0) != expected_out[target]:
            raise ValueError(f"Target {target!r} expects output dim {expected_out[target]}, got {b.size(0)}")
        if b.size(1) < effective_rank:
            raise ValueError(f"Target {target!r} rank dim {b.size(1)} is smaller than effective_rank={effective_rank}")


def _check_single_payload(name, lora_a, lora_b, effective_rank, in_dim, out_dim) -> None:
    if isinstance(lora_b, list):
        raise ValueError(f"{name} expects tensor lora_b")
    if lora_a.ndim != 2:
        raise ValueError(f"{name} expects 2D lora_a, got shape={tuple(lora_a.shape)}")
    if lora_b.ndim != 2:
        raise ValueError(f"{name} expects 2D lora_b, got shape={tuple(lora_b.shape)}")
    if lora_a.size(0) < effective_rank:
        raise ValueError(f"LoRA A rank dim {lora_a.size(0)} is smaller than effective_rank={effective_rank}")
    if lora_a.size(1) != in_dim:
        raise ValueError(f"Expected lora_a input dim {in_dim}, got {lora_a.size(1)}")
    if lora_b.size(0) != out_dim:
        raise ValueError(f"Expected lora_b output dim {out_dim}, got {lora_b.size(0)}")
    if lora_b.size(1) < effective_rank:
        raise ValueError(f"LoRA B rank dim {lora_b.size(1)} is smaller than effective_rank={effective_rank}")


class LoRAQKVParallelLinear(_LoRALayerBase):
    """Column-parallel fused q/k/v projection; ``lora_B_*`` are sharded on the output
    dim like the base weight, ``lora_A`` is replicated (no LoRA collective)."""

    _ORDER = ("q", "k", "v")

    def __init__(
        self,
        hidden_size: int,
        head_size: int,
        total_num_heads: int,
        total_num_kv_heads: int,
        bias: bool = False,
        lora_targets: Optional[list[str]] = None,
        max_loras: int = 1,
        max_lora_rank: int | None = None,
        lora_domain: str = LM_LORA_DOMAIN,
    ):
        rank = max_lora_rank or 0
        targets = list(lora_targets) if lora_targets else list(self._ORDER)
        super().__init__(max_loras, rank, rank > 0 and len(targets) > 0, lora_domain)
        self.tp_size, self.tp_rank = _get_world_size(), _get_rank()
        self.hidden_size, self.head_size = hidden_size, head_size
        self.total_num_heads, self.total_num_kv_heads = total_num_heads, total_num_kv_heads
        self.num_heads = divide(total_num_heads, self.tp_size)
        self.num_kv_heads = divide(total_num_kv_heads, self.tp_size)
        self.q_size = self.num_heads * head_size
        self.kv_size = self.num_kv_heads * head_size
        out = self.q_size + 2 * self.kv_size
        self.weight = nn.Parameter(torch.empty(out, hidden_size))
        self.bias = nn.Parameter(torch.empty(out)) if bias else None
        self.lora_targets = targets
        self.target_to_index = {t: i for i, t in enumerate(targets)}
        if self.supports_lora:
            self.lora_A = nn.Parameter(torch.zeros(len(targets), max_loras, rank, hidden_size))
            for t in targets:
                setattr(self, f"lora_B_{t}", nn.Parameter(torch.zeros(max_loras, self._width(t), rank)))

    def _width(self, target: str) -> int:
        return self.q_size if target == "q" else self.kv_size

    def _column(self, target: str) -> int:
        return {"q": 0, "k": self.q_size, "v": self.q_size + self.kv_size}[target]

    def _a_slices(self):
        return [self.lora_A[i] for i in range(len(self.lora_targets))]

    def _b_slices(self):
        return [getattr(self, f"lora_B_{t}") for t in self.lora_targets]

    def _slice_layout(self):
        return [self._width(t) for t in self.lora_targets], [self._column(t) for t in self.lora_targets]

    def load_base_shard(self, loaded_weight: torch.Tensor, shard_id: str) -> None:
        """Copy this rank's rows of a full q / k / v weight into the packed weight."""
        rows = self._width(shard_id)
        self.weight.data.narrow(0, self._column(shard_id), rows).copy_(
            loaded_weight.chunk(self.tp_size, 0)[self.tp_rank]
        )

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._linear(x, self.weight, self.bias)

    def set_slot_lora(self, slot_id, lora_a, lora_b, effective_rank, scaling) -> None:
        self._write_slot(slot_id, list(lora_a), list(lora_b), effective_rank, scaling)

    def validate_slot_lora_payload(self, lora_a, lora_b, effective_rank, scaling) -> None:
        self._validate_common_slot_payload(effective_rank, scaling)
        _check_multi_payload(
            "LoRAQKVParallelLinear", self.lora_targets, lora_a, lora_b, effective_rank, self.hidden_size,
            {"q": self.q_size, "k": self.kv_size, "v": self.kv_size},
        )


class LoRAMergedColumnParallelLinear(_LoRALayerBase):
    """Column-parallel merged projection (gate / up), one LoRA slice per merged output."""

    def __init__(
        self,
        input_size: int,
        output_sizes: list[int],
        bias: bool = False,
        lora_targets: Optional[list[int]] = None,
        max_loras: int = 1,
        max_lora_rank: int | None = None,
        lora_domain: str = LM_LORA_DOMAIN,
    ):
        rank = max_lora_rank or 0
        targets = list(lora_targets) if lora_targets is not None else list(range(len(output_sizes)))
        super().__init__(max_loras, rank, rank > 0 and len(targets) > 0, lora_domain)
        self.tp_size, self.tp_rank = _get_world_size(), _get_rank()
        self.input_size, self.output_sizes = input_size, output_sizes
        self.shard_output_sizes = [s // self.tp_size for s in output_sizes]
        out = sum(output_sizes) // self.tp_size
        self.weight = nn.Parameter(torch.empty(out, input_size))
        self.bias = nn.Parameter(torch.empty(out)) if bias else None
        self.lora_targets = targets
        self.target_to_index = {t: i for i, t in enumerate(targets)}
        if self.supports_lora:
            self.lora_A = nn.Parameter(torch.zeros(len(targets), max_loras, rank, input_size))
            for t in targets:
                setattr(self, f"lora_B_{t}", nn.Parameter(torch.zeros(max_loras, self.shard_output_sizes[t], rank)))

    def _a_slices(self):
        return [self.lora_A[i] for i in range(len(self.lora_targets))]

    def _b_slices(self):
        return [getattr(self, f"lora_B_{t}") for t in self.lora_targets]

    def _slice_layout(self):
        starts = [sum(self.shard_output_sizes[:t]) for t in self.lora_targets]
        return [self.shard_output_sizes[t] for t in self.lora_targets], starts

    def load_base_shard(self, loaded_weight: torch.Tensor, shard_id: int) -> None:
        start = sum(self.shard_output_sizes[:shard_id])
        self.weight.data.narrow(0, start, self.shard_output_sizes[shard_id]).copy_(
            loaded_weight.chunk(self.tp_size, 0)[self.tp_rank]
        )

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._linear(x, self.weight, self.bias)

    def set_slot_lora(self, slot_id, lora_a, lora_b, effective_rank, scaling) -> None:
        self._write_slot(slot_id, list(lora_a), list(lora_b), effective_rank, scaling)

    def validate_slot_lora_payload(self, lora_a, lora_b, effective_rank, scaling) -> None:
        self._validate_common_slot_payload(effective_rank, scaling)
        _check_multi_payload(
            "LoRAMergedColumnParallelLinear", self.lora_targets, lora_a, lora_b, effective_rank, self.input_size,
            {t: self.shard_output_sizes[t] for t in self.lora_targets},
        )


class LoRARowParallelLinear(_LoRALayerBase):
    """Row-parallel projection (o / down).

    ``lora_tp_mode``:
      * ``"partial_y"`` (reference semantics, ``layers/lora.py:722-742``): ``lora_A`` is
        sharded on the input dim, ``lora_B`` is full on every rank, each rank adds its
        partial delta to its partial ``y`` and the one ``[T, out]`` all-reduce sums both.
      * ``"allreduce_tmp"``: the fp32 shrink result ``[T, r]`` is all-reduced instead
        (``out / r`` times fewer bytes than a second ``[T, out]`` exchange would need),
        after which every rank expands only its ``out / tp`` columns of a ``lora_B`` that
        is sharded on the output dim; the base all-reduce assembles the delta exactly once.
      * ``"peer_exchange"``: as ``"allreduce_tmp"``, but the ``[T, r]`` sum is one kernel over
        peer memory (``tp_exchange.TpExchange`` assigned to ``self.tp_exchange``, shared by the
        layers of a model) instead of a library collective.
    """

    def __init__(
        self,
        input_size: int,
        output_size: int,
        bias: bool = False,
        max_loras: int = 1,
        max_lora_rank: int | None = None,
        lora_domain: str = LM_LORA_DOMAIN,
        lora_tp_mode: str = "partial_y",
    ):
        rank = max_lora_rank or 0
        super().__init__(max_loras, rank, rank > 0, lora_domain)
        if lora_tp_mode not in ("partial_y", "allreduce_tmp", "peer_exchange"):
            raise ValueError(f"unknown lora_tp_mode {lora_tp_mode!r}")
        self.tp_size, self.tp_rank = _get_world_size(), _get_rank()
        self.input_size, self.output_size = input_size, output_size
        self.shard_input_size = divide(input_size, self.tp_size)
        self.lora_tp_mode = lora_tp_mode if self.tp_size > 1 else "partial_y"
        self.tp_exchange = None  # TpExchange for "peer_exchange", assigned by whoever builds the model
        self.weight = nn.Parameter(torch.empty(output_size, self.shard_input_size))
        self.bias = nn.Parameter(torch.empty(output_size)) if bias else None
        if self.supports_lora:
            self.lora_A = nn.Parameter(torch.zeros(max_loras, rank, self.shard_input_size))
            b_rows = output_size if self.lora_tp_mode == "partial_y" else divide(output_size, self.tp_size)
            self.lora_B = nn.Parameter(torch.zeros(max_loras, b_rows, rank))

    def _a_slices(self):
        return [self.lora_A]

    def _b_slices(self):
        return [self.lora_B]

    def _slice_layout(self):
        if self.lora_tp_mode != "partial_y":
            w = self.output_size // self.tp_size
            return [w], [self.tp_rank * w]
        return [self.output_size], [0]

    def load_base_shard(self, loaded_weight: torch.Tensor) -> None:
        self.weight.data.copy_(loaded_weight.narrow(1, self.tp_rank * self.shard_input_size, self.shard_input_size))

    def _apply_lora_allreduce_tmp(self, y: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        from .lora import SGMV_MIN_TOKENS
        from .lora_ops import expand_into, shrink_into

        if self._per_part(self._apply_lora_allreduce_tmp, y, x) is not None:
            return y
        x_flat = x if x.dim() == 2 else x.reshape(-1, x.size(-1))
        token_to_slot = self._resolve_token_slots(x_flat)
        if token_to_slot is None:
            return y
        y_flat = y if y.dim() == 2 else y.view(-1, y.size(-1))
        # prefill-sized bf16 batches: both halves on the tensor-core kernels around a bf16 [T, r] sum
        # (rows of one adapter must be contiguous for those: a batch with fewer than 32 rows per adapter bucket is a
        # decode batch, whatever its size, and stays on the bucket kernel)
        meta = self._runtime_metadata()
        scattered = meta is not None and meta.num_active_loras > 0 and x_flat.size(0) < 32 * meta.num_active_loras
        tensor_core = (x.is_cuda and x.dtype == torch.bfloat16 and x_flat.size(0) >= SGMV_MIN_TOKENS and not scattered
                       and self.max_lora_rank in (16, 32, 64) and x_flat.size(1) % 64 == 0)
        if self.lora_tp_mode == "peer_exchange" and x.is_cuda and not tensor_core:
            # one C call: bucket kernel (shrink half) -> peer-memory exchange -> bucket kernel (expand half)
            if self.tp_exchange is None:
                raise RuntimeError("lora_tp_mode='peer_exchange' needs a TpExchange in layer.tp_exchange")
            metadata = self._runtime_metadata()
            if metadata is None:
                raise RuntimeError("LoRA metadata must be prepared by the model runner before backend execution")
            widths, cols = self._slice_layout()
            self.tp_exchange.row_parallel_add(y_flat, x_flat, [self.lora_A], [self.lora_B], widths, cols, metadata, 1.0,
                                              rank_per_slot=self.effective_lora_rank)
            return y
        tmp = torch.empty((1, x_flat.size(0), self.max_lora_rank), dtype=torch.bfloat16 if tensor_core else torch.float32,
                          device=x.device)
        shrink_into(tmp, x_flat, [self.lora_A], token_to_slot, 1.0)
        if self.lora_tp_mode == "peer_exchange" and not tensor_core:
            if self.tp_exchange is None:
                raise RuntimeError("lora_tp_mode='peer_exchange' needs a TpExchange in layer.tp_exchange")
            self.tp_exchange.all_reduce_(tmp)  # one kernel over peer memory
        else:
            dist.all_reduce(tmp)  # [T, r] fp32 partials over the input shards
        widths, cols = self._slice_layout()
        expand_into(y_flat, tmp, [self.lora_B], token_to_slot, offset_start=cols[0], add_inputs=True)
        return y

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        bias = self.bias if self.tp_rank == 0 else None
        if self.lora_tp_mode != "partial_y":
            y = self._apply_lora_allreduce_tmp(F.linear(x, self.weight, bias), x)
        else:
            y = self._linear(x, self.weight, bias)
        if self.tp_size > 1:
            dist.all_reduce(y)
        return y

    def set_slot_lora(self, slot_id, lora_a, lora_b, effective_rank, scaling) -> None:
        self._write_slot(slot_id, [lora_a], [lora_b], effective_rank, scaling)

    def validate_slot_lora_payload(self, lora_a, lora_b, effective_rank, scaling) -> None:
        self._validate_common_slot_payload(effective_rank, scaling)
        _check_single_payload(
            "LoRARowParallelLinear", lora_a, lora_b, effective_rank, self.shard_input_size, self.lora_B.size(1)
        )


class LoRALinear(_LoRALayerBase):
    """Un-sharded linear (+bias) with one LoRA slice."""

    def __init__(
        self,
        in_features: int,
        out_features: int,
        bias: bool = True,
        max_loras: int = 1,
        max_lora_rank: int | None = None,
        lora_domain: str = LM_LORA_DOMAIN,
    ):
        rank = max_lora_rank or 0
        super().__init__(max_loras, rank, rank > 0, lora_domain)
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.empty(out_features)) if bias else None
        if self.supports_lora:
            self.lora_A = nn.Parameter(torch.zeros(max_loras, rank, in_features))
            self.lora_B = nn.Parameter(torch.zeros(max_loras, out_features, rank))

    def _a_slices(self):
        return [self.lora_A]

    def _b_slices(self):
        return [self.lora_B]

    def _slice_layout(self):
        return [self.out_features], [0]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._linear(x, self.weight, self.bias)

    def set_slot_lora(self, slot_id, lora_a, lora_b, effective_rank, scaling) -> None:
        self._write_slot(slot_id, [lora_a], [lora_b], effective_rank, scaling)

    def validate_slot_lora_payload(self, lora_a, lora_b, effective_rank, scaling) -> None:
        self._validate_common_slot_payload(effective_rank, scaling)
        _check_single_payload("LoRALinear", lora_a, lora_b, effective_rank, self.in_features, self.out_features)


_LORA_LAYER_TYPES = (LoRAQKVParallelLinear, LoRAMergedColumnParallelLinear, LoRARowParallelLinear, LoRALinear)


def iter_lora_modules(model: nn.Module):
    for module in model.modules():
        if isinstance(module, _LORA_LAYER_TYPES) and module.lora_enabled:
            yield module


def get_lora_state_dict(model: nn.Module) -> dict:
    return {name: p.data.clone() for name, p in model.named_parameters() if "lora_" in name}
