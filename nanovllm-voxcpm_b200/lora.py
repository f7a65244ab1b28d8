"""Operator API of the multi-LoRA linear path, backed by the sm_100a C-ABI library.

Mirrors the reference's ``nanovllm_voxcpm/lora.py``: the ``LoRABackend`` protocol
(``lora.py:40-58``), ``LoRAMetadata`` (``lora.py:18-37``), ``LoRAAvailability``
(``lora.py:12-15``) and the backend selection helpers (``lora.py:414-439``).
``B200LoRABackend`` takes the place of ``_VendoredTritonPunicaBackend``
(``lora.py:121-399``): same arguments, same in-place / return contract, same
exceptions before launch, but one fused CUDA launch per call instead of
memset + shrink + stack + expand.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Protocol

import torch

from . import _native as N


@dataclass(frozen=True)
class LoRAAvailability:
    available: bool
    reason: str | None = None


@dataclass(frozen=True)
class LoRAMetadata:
    """Index bundle of one step (all int32, on the execution device).

    ``token_to_slot[T]`` is the only mandatory tensor; the bucket arrays
    (``token_indices_sorted_by_slot``, ``active_slot_ids``, ``num_tokens_per_slot``,
    ``slot_start_offsets``) enable the grouped kernels.  All three conventions of
    the reference are accepted: the eager batch plan (only slots >= 0), the CUDA
    graph buffers (leading ``-1`` bucket with count 0, ``max_loras + 1`` buckets)
    and the vLLM-style layout (``-1`` bucket with its real count).
    """

    token_to_slot: torch.Tensor | None
    token_indices_sorted_by_slot: torch.Tensor | None
    active_slot_ids: torch.Tensor | None
    num_tokens_per_slot: torch.Tensor | None
    slot_start_offsets: torch.Tensor | None
    no_lora_flag: bool
    num_active_loras: int = 0

    def as_kernel_metadata(self, token_count: int):
        cut = lambda t: None if t is None else t[:token_count]  # noqa: E731
        return (
            cut(self.token_to_slot),
            cut(self.token_indices_sorted_by_slot),
            self.num_tokens_per_slot,
            self.slot_start_offsets,
            self.active_slot_ids,
            self.no_lora_flag,
            self.num_active_loras,
        )


class LoRABackend(Protocol):
    def availability(self) -> LoRAAvailability: ...

    def add_lora(
        self,
        y_slices: list[torch.Tensor],
        x: torch.Tensor,
        lora_a_slices: list[torch.Tensor],
        lora_b_slices: list[torch.Tensor],
        *,
        indices: torch.Tensor,
        metadata: LoRAMetadata | None,
        scaling: float,
        y_packed: torch.Tensor | None = None,
    ) -> list[torch.Tensor]: ...

    def shrink(self, x: torch.Tensor, lora_a: torch.Tensor) -> torch.Tensor: ...

    def expand(self, hidden: torch.Tensor, lora_b: torch.Tensor, *, scaling: float) -> torch.Tensor: ...


def _as_3d(slab: torch.Tensor) -> torch.Tensor:
    # [S, 1, a, b] slabs are accepted like the reference's pointer helpers do
    # (lora_ops/triton_ops/utils.py:25-29,65-69).
    if slab.dim() == 4 and slab.size(1) == 1:
        return slab.squeeze(1)
    if slab.dim() != 3:
        raise ValueError(f"LoRA slab must be [slots, a, b] (or [slots, 1, a, b]); got shape {tuple(slab.shape)}")
    return slab


def _i32(t: torch.Tensor | None, name: str) -> torch.Tensor | None:
    if t is None:
        return None
    if t.dtype != torch.int32:
        raise ValueError(f"LoRA metadata tensor {name} must be int32, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"LoRA metadata tensor {name} must be contiguous")
    return t


#: batches of at least this many rows use the tensor-core prefill kernels under IMPL_AUTO
SGMV_MIN_TOKENS = 512

_SCRATCH: dict[torch.device, torch.Tensor] = {}
#: buffers that were replaced by a larger one: a CUDA graph captured earlier may still write through their
#: addresses, so they are kept for the life of the process instead of going back to the allocator
_RETIRED_SCRATCH: list[torch.Tensor] = []


def reserve_scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    """Sizes the per-device scratch buffer up front (e.g. from ``max_num_batched_tokens`` x slices x
    ``max_lora_rank`` before CUDA graphs are captured), so that it never has to grow later."""
    return scratch_for(torch.device(device), int(nbytes))


def scratch_for(device: torch.device, nbytes: int) -> torch.Tensor:
    """Per-device scratch buffer for the prefill kernels' rank-r intermediate.

    The reference allocates this intermediate on every call (``lora.py:302``); here one buffer per device
    is reused, so steady-state calls (and CUDA-graph replays) allocate nothing. The buffer only grows, and a
    buffer that is outgrown is never freed: its address may be baked into a captured graph. One buffer per
    device means one stream at a time may run calls that use it (the runner's single stream); callers that
    overlap streams pass their own ``workspace``."""
    buf = _SCRATCH.get(device)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _RETIRED_SCRATCH.append(buf)
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _SCRATCH[device] = buf
    return buf


def launch_add(
    y_packed: torch.Tensor,
    x: torch.Tensor,
    a_slabs: list[torch.Tensor],
    b_slabs: list[torch.Tensor],
    out_sizes: list[int],
    col_offsets: list[int],
    metadata: LoRAMetadata,
    scaling: float,
    *,
    rank_per_slot: torch.Tensor | None = None,
    scale_per_slot: torch.Tensor | None = None,
    impl: int = N.IMPL_AUTO,
    workspace: torch.Tensor | None = None,
    overwrite: bool = False,
) -> None:
    """One ``lora_b200_add`` call: all slices share (slots, rank, in). ``overwrite=True`` is ``lora_b200_delta``:
    ``y_packed`` receives the delta (and -0.0 in rows without one) instead of being added to."""
    T = x.size(0)
    N.require_cuda(y_packed, x, *a_slabs, *b_slabs, metadata.token_to_slot)
    if y_packed.dim() != 2 or x.dim() != 2:
        raise ValueError("x and y must be 2D [num_tokens, features]")
    if x.stride(1) != 1 or y_packed.stride(1) != 1:
        raise ValueError("x and y must have unit column stride")
    dt = N.dtype_code(x.dtype)
    for t in (y_packed, *a_slabs, *b_slabs):
        if t.dtype != x.dtype:
            raise ValueError(f"x, y and the LoRA slabs must share one dtype; got {x.dtype} and {t.dtype}")
    S, r_max, in_dim = a_slabs[0].shape
    if in_dim != x.size(1):
        raise ValueError(f"lora_A input dim {in_dim} does not match x features {x.size(1)}")
    tts, srt, cnt, off, ids, _, _ = metadata.as_kernel_metadata(T)
    tts = _i32(tts, "token_to_slot")
    if tts is None or tts.numel() != T:
        raise RuntimeError(
            "LoRA token_to_slot length does not match input rows: "
            f"token_to_slot={0 if tts is None else tts.numel()} rows={T}"
        )
    if tts.device != x.device:
        raise RuntimeError("LoRA token_to_slot must be prepared on the execution device by the model runner")
    srt, ids, cnt, off = _i32(srt, "sorted"), _i32(ids, "slot ids"), _i32(cnt, "counts"), _i32(off, "offsets")
    n_buckets = 0
    if srt is not None and ids is not None and cnt is not None and off is not None:
        n_buckets = min(ids.numel(), cnt.numel(), off.numel() - 1)
        if metadata.num_active_loras > 0:
            n_buckets = min(n_buckets, metadata.num_active_loras)
    if n_buckets <= 0:
        srt = ids = cnt = off = None
        n_buckets = 0
    if workspace is None and x.dtype == torch.bfloat16 and (
        impl == N.IMPL_SGMV or (impl == N.IMPL_AUTO and T >= SGMV_MIN_TOKENS)
    ):
        workspace = scratch_for(x.device, N.workspace_bytes(T, len(a_slabs), r_max))
    with N.on_device(x.device):
        rc = (N.lib().lora_b200_delta if overwrite else N.lib().lora_b200_add)(
            y_packed.data_ptr(), y_packed.stride(0), x.data_ptr(), x.stride(0), T, in_dim, len(a_slabs),
            N.ptr_array(a_slabs), N.ptr_array(b_slabs), N.int_array(out_sizes), N.int_array(col_offsets),
            S, r_max, N.ptr(rank_per_slot), N.ptr(scale_per_slot), tts.data_ptr(), N.ptr(srt), N.ptr(ids),
            N.ptr(cnt), N.ptr(off), n_buckets, float(scaling), dt, impl,
            N.ptr(workspace), 0 if workspace is None else workspace.numel() * workspace.element_size(),
            N.current_stream(x.device),
        )
    N.check(rc)


def fused_linear_supported(x: torch.Tensor, weight: torch.Tensor, r_max: int) -> bool:
    """Shapes / dtypes the fused base-GEMM + LoRA kernel takes (bf16, in % 64 == 0, rank 16/32/64)."""
    return (
        x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
        and x.size(1) % 64 == 0 and weight.size(0) % 8 == 0 and weight.stride(1) == 1 and x.stride(1) == 1
        and r_max in (16, 32, 64)
    )


def linear_lora(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None,
    a_slabs: list[torch.Tensor],
    b_slabs: list[torch.Tensor],
    out_sizes: list[int],
    col_offsets: list[int],
    token_to_slot: torch.Tensor | None,
    scaling: float = 1.0,
    *,
    scale_per_slot: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """``x @ weight.T (+ bias)`` plus the multi-LoRA delta in one pass over the output
    (``lora_b200_linear_lora``): what the reference computes as ``F.linear`` followed by
    ``add_lora`` (``layers/lora.py:341-366``). ``token_to_slot=None`` gives the plain linear."""
    N.require_cuda(x, weight, bias, token_to_slot, *a_slabs, *b_slabs)
    T, in_dim = x.shape
    out_total = weight.size(0)
    if out is None:
        out = torch.empty((T, out_total), dtype=x.dtype, device=x.device)
    if weight.size(1) != in_dim:
        raise ValueError(f"weight input dim {weight.size(1)} does not match x features {in_dim}")
    n = len(a_slabs) if token_to_slot is not None else 0
    S = r_max = 1
    workspace = None
    if n:
        a_slabs = [_as_3d(a) for a in a_slabs]
        b_slabs = [_as_3d(b) for b in b_slabs]
        S, r_max, a_in = a_slabs[0].shape
        if a_in != in_dim:
            raise ValueError(f"lora_A input dim {a_in} does not match x features {in_dim}")
        if token_to_slot.dtype != torch.int32 or token_to_slot.numel() != T:
            raise RuntimeError(
                f"LoRA token_to_slot length does not match input rows: token_to_slot={token_to_slot.numel()} rows={T}"
            )
        workspace = scratch_for(x.device, N.workspace_bytes(T, n, r_max))
    with N.on_device(x.device):
        rc = N.lib().lora_b200_linear_lora(
            out.data_ptr(), out.stride(0), x.data_ptr(), x.stride(0), T, in_dim, weight.data_ptr(), weight.stride(0),
            out_total, N.ptr(bias), n, N.ptr_array(a_slabs[:n]) if n else None, N.ptr_array(b_slabs[:n]) if n else None,
            N.int_array(out_sizes[:n]) if n else None, N.int_array(col_offsets[:n]) if n else None, S, r_max,
            N.ptr(scale_per_slot), N.ptr(token_to_slot) if n else None, float(scaling), N.ptr(workspace),
            0 if workspace is None else workspace.numel(), N.current_stream(x.device),
        )
    N.check(rc)
    return out


class B200LoRABackend:
    """``LoRABackend`` on hand-written sm_100a kernels (no Triton, no CPU path)."""

    def __init__(self, impl: int = N.IMPL_AUTO) -> None:
        self.impl = impl
        self._zero_index: dict[tuple[torch.device, int], torch.Tensor] = {}

    # ---------------------------------------------------------------- probing
    def availability(self) -> LoRAAvailability:
        if not torch.cuda.is_available():
            return LoRAAvailability(False, "CUDA is unavailable")
        try:
            N.lib()
        except (OSError, AttributeError, N.NativeLibraryError) as exc:
            return LoRAAvailability(False, f"B200 LoRA library unavailable: {exc}")
        major, _ = torch.cuda.get_device_capability()
        if major != 10:
            return LoRAAvailability(False, f"kernels are built for sm_100a only; device is sm_{major}x")
        return LoRAAvailability(True, None)

    def prime_slice_caches(self, lora_a_slices, lora_b_slices, *, offset_start: int = 0) -> None:
        """Nothing to prime: slab pointers travel by value in the launch parameters,
        so there is no device pointer table to allocate before CUDA-graph capture
        (the reference needs this step, ``lora.py:134-178``)."""
        return None

    # --------------------------------------------------------------- add_lora
    def add_lora(
        self,
        y_slices: list[torch.Tensor],
        x: torch.Tensor,
        lora_a_slices: list[torch.Tensor],
        lora_b_slices: list[torch.Tensor],
        *,
        indices: torch.Tensor,
        metadata: LoRAMetadata | None,
        scaling: float,
        y_packed: torch.Tensor | None = None,
        rank_per_slot: torch.Tensor | None = None,
        scale_per_slot: torch.Tensor | None = None,
    ) -> list[torch.Tensor]:
        """``y[t, slice] += scaling * (x[t] @ A[slot_t].T) @ B[slot_t].T`` for slot_t >= 0.

        Contract of the reference (``lora.py:241-381``): with ``y_packed`` (or a
        single slice) the update is in place and the same views come back; several
        slices without ``y_packed`` are concatenated into a new buffer whose column
        views are returned and the inputs stay untouched.  ``indices`` is accepted
        for signature compatibility; routing comes from ``metadata`` exactly as in
        the reference (``lora.py:291``).  ``rank_per_slot`` / ``scale_per_slot`` are
        optional extensions (device int32 / float32 ``[slots]``).
        """
        if not y_slices:
            return []
        if len(y_slices) != len(lora_a_slices) or len(y_slices) != len(lora_b_slices):
            raise ValueError("add_lora expects aligned y/lora_a/lora_b slice lists")
        if metadata is None:
            raise RuntimeError("LoRA metadata must be prepared by the model runner before backend execution")
        if not all(t.is_contiguous() for t in lora_a_slices):
            raise ValueError("add_lora expects contiguous lora_a slices")
        if not all(t.is_contiguous() for t in lora_b_slices):
            raise ValueError("add_lora expects contiguous lora_b slices")

        if y_packed is None:
            if len(y_slices) == 1:
                y_packed = y_slices[0]
            else:
                widths = [y.size(-1) for y in y_slices]
                y_packed = torch.cat(y_slices, dim=-1)
                y_slices = list(y_packed.split(widths, dim=-1))
        elif y_packed.dim() != 2:
            raise ValueError("y_packed must be 2D [num_tokens, packed_hidden]")

        if metadata.no_lora_flag or x.size(0) == 0:
            return list(y_slices)

        a3 = [_as_3d(a) for a in lora_a_slices]
        b3 = [_as_3d(b) for b in lora_b_slices]
        widths = [y.size(-1) for y in y_slices]
        offsets = [0]
        for w in widths:
            offsets.append(offsets[-1] + w)
        for i, (a, b) in enumerate(zip(a3, b3)):
            if b.size(1) != widths[i] and widths[i] > 0:
                raise ValueError(f"slice {i}: lora_B rows {b.size(1)} != output width {widths[i]}")
            if b.size(2) != a.size(1) or b.size(0) != a.size(0):
                raise ValueError(f"slice {i}: lora_A {tuple(a.shape)} and lora_B {tuple(b.shape)} disagree")

        # one launch per (slots, rank, in) group; in the layers all slices share it
        groups: dict[tuple[int, int, int], list[int]] = {}
        for i, a in enumerate(a3):
            if widths[i] == 0:
                continue  # a TP shard that owns no rows of this slice (lora.py:209,215)
            groups.setdefault(tuple(a.shape), []).append(i)
        for members in groups.values():
            for k in range(0, len(members), N.MAX_SLICES):
                part = members[k : k + N.MAX_SLICES]
                launch_add(
                    y_packed, x, [a3[i] for i in part], [b3[i] for i in part], [widths[i] for i in part],
                    [offsets[i] for i in part], metadata, scaling, rank_per_slot=rank_per_slot,
                    scale_per_slot=scale_per_slot, impl=self.impl,
                )
        return list(y_slices)

    # -------------------------------------------------- single-adapter helpers
    def _zeros_index(self, device: torch.device, T: int) -> torch.Tensor:
        key = (device, T)
        idx = self._zero_index.get(key)
        if idx is None:
            idx = torch.zeros(T, dtype=torch.int32, device=device)
            self._zero_index[key] = idx
        return idx

    def shrink(self, x: torch.Tensor, lora_a: torch.Tensor) -> torch.Tensor:
        """``x @ lora_a.T`` for one adapter ``[r, in]`` -> ``[T, r]``
        (meaning fixed by the reference's test backends, tests/unit/test_lora_layers.py:12-13)."""
        from .lora_ops import shrink_into

        N.require_cuda(x, lora_a)
        out = torch.empty((1, x.size(0), lora_a.size(0)), dtype=x.dtype, device=x.device)
        shrink_into(out, x, [lora_a.contiguous().unsqueeze(0)], self._zeros_index(x.device, x.size(0)), 1.0)
        return out.squeeze(0)

    def expand(self, hidden: torch.Tensor, lora_b: torch.Tensor, *, scaling: float) -> torch.Tensor:
        """``(hidden @ lora_b.T) * scaling`` for one adapter ``[out, r]`` -> ``[T, out]``, not accumulated
        (tests/unit/test_lora_layers.py:15-16)."""
        from .lora_ops import expand_into

        N.require_cuda(hidden, lora_b)
        out = torch.empty((hidden.size(0), lora_b.size(0)), dtype=hidden.dtype, device=hidden.device)
        expand_into(
            out, hidden.contiguous().unsqueeze(0), [lora_b.contiguous().unsqueeze(0)],
            self._zeros_index(hidden.device, hidden.size(0)), offset_start=0, add_inputs=False,
        )
        return out * scaling


class _UnavailableBackend:
    def __init__(self, reason: str):
        self.reason = reason

    def availability(self) -> LoRAAvailability:
        return LoRAAvailability(False, self.reason)

    def add_lora(self, *args, **kwargs):
        raise RuntimeError(self.reason)

    def shrink(self, *args, **kwargs):
        raise RuntimeError(self.reason)

    def expand(self, *args, **kwargs):
        raise RuntimeError(self.reason)


_BACKEND_OVERRIDE: LoRABackend | None = None
_PROBED_BACKEND: LoRABackend | None = None


def get_backend() -> LoRABackend:
    """Override if set, else the probed B200 backend; an unavailable backend raises
    ``RuntimeError`` with the reason on use - there is no other implementation."""
    global _PROBED_BACKEND
    if _BACKEND_OVERRIDE is not None:
        return _BACKEND_OVERRIDE
    if _PROBED_BACKEND is None:
        backend = B200LoRABackend()
        status = backend.availability()
        _PROBED_BACKEND = backend if status.available else _UnavailableBackend(status.reason or "unavailable")
    return _PROBED_BACKEND


def set_backend_for_testing(backend: LoRABackend | None) -> None:
    global _BACKEND_OVERRIDE
    _BACKEND_OVERRIDE = backend


def get_availability() -> LoRAAvailability:
    return get_backend().availability()


def is_available() -> bool:
    return get_availability().available


def assert_available() -> None:
    status = get_availability()
    if not status.available:
        raise RuntimeError(status.reason or "LoRA runtime is unavailable")


def install_into_reference(backend: LoRABackend | None = None) -> LoRABackend:
    """Make the reference package route its LoRA layers through this backend.

    Uses the reference's own hook (``nanovllm_voxcpm.lora.set_backend_for_testing``,
    ``lora.py:423-425``); requires ``nanovllm_voxcpm`` to be importable.
    """
    import nanovllm_voxcpm.lora as ref_lora

    backend = backend or B200LoRABackend()
    ref_lora.set_backend_for_testing(backend)
    return backend
