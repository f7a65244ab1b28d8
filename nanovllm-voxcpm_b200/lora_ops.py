"""``lora_shrink`` / ``lora_expand`` / ``LoRAKernelMeta`` with the reference's signatures.

Drop-in for ``nanovllm_voxcpm/lora_ops/__init__.py:1-5``: the two free functions keep
the positional arguments of ``lora_ops/triton_ops/lora_shrink_op.py:258-270`` and
``lora_expand_op.py:95-108``; ``LoRAKernelMeta`` keeps the field names and the
vLLM-style bucket layout of ``lora_ops/triton_ops/lora_kernel_metadata.py:9-79``.
"""

from __future__ import annotations

import bisect
from dataclasses import dataclass, field

import torch

from . import _native as N


def _slab3(t: torch.Tensor) -> torch.Tensor:
    if t.dim() == 4 and t.size(1) == 1:
        t = t.squeeze(1)
    if t.dim() != 3:
        raise ValueError(f"LoRA slab must be 3D [slots, a, b]; got {tuple(t.shape)}")
    if not t.is_contiguous():
        raise ValueError("LoRA slabs must be contiguous")
    return t


def shrink_into(
    output_tensor: torch.Tensor,
    inputs: torch.Tensor,
    lora_a_weights: list[torch.Tensor],
    token_lora_mapping: torch.Tensor,
    scaling: float,
) -> None:
    slabs = [_slab3(a) for a in lora_a_weights]
    N.require_cuda(output_tensor, inputs, token_lora_mapping, *slabs)
    S, r, in_dim = slabs[0].shape
    T = inputs.size(0)
    if any(tuple(a.shape) != (S, r, in_dim) for a in slabs):
        raise ValueError("lora_shrink expects lora_a slices of one shape")
    if tuple(output_tensor.shape) != (len(slabs), T, r) or not output_tensor.is_contiguous():
        raise ValueError(f"lora_shrink output must be contiguous [{len(slabs)}, {T}, {r}]")
    if inputs.dim() != 2 or inputs.stride(1) != 1 or inputs.size(1) != in_dim:
        raise ValueError("lora_shrink input must be [tokens, in] with unit column stride")
    if token_lora_mapping.dtype != torch.int32 or token_lora_mapping.numel() < T:
        raise ValueError("token_lora_mapping must be int32 with one entry per token")
    with N.on_device(inputs.device):
        rc = N.lib().lora_b200_shrink(
            output_tensor.data_ptr(), N.dtype_code(output_tensor.dtype), inputs.data_ptr(), inputs.stride(0), T,
            in_dim, len(slabs), N.ptr_array(slabs), S, r, token_lora_mapping.data_ptr(), float(scaling),
            N.dtype_code(inputs.dtype), N.current_stream(inputs.device),
        )
    N.check(rc)


def expand_into(
    output_tensor: torch.Tensor,
    inputs: torch.Tensor,
    lora_b_weights: list[torch.Tensor],
    token_lora_mapping: torch.Tensor,
    *,
    offset_start: int,
    add_inputs: bool,
) -> None:
    slabs = [_slab3(b) for b in lora_b_weights]
    N.require_cuda(output_tensor, inputs, token_lora_mapping, *slabs)
    S, _, r = slabs[0].shape
    T = inputs.size(1)
    if inputs.dim() != 3 or tuple(inputs.shape) != (len(slabs), T, r) or not inputs.is_contiguous():
        raise ValueError(f"lora_expand input must be contiguous [{len(slabs)}, tokens, {r}]")
    if any(b.size(0) != S or b.size(2) != r for b in slabs):
        raise ValueError("lora_expand expects lora_b slices with one (slots, rank)")
    if output_tensor.dim() != 2 or output_tensor.stride(1) != 1 or output_tensor.size(0) != T:
        raise ValueError("lora_expand output must be [tokens, hidden] with unit column stride")
    widths = [b.size(1) for b in slabs]
    cols = [offset_start]
    for w in widths[:-1]:
        cols.append(cols[-1] + w)
    if cols[-1] + widths[-1] > output_tensor.size(1):
        raise ValueError("lora_expand slices exceed the output width")
    with N.on_device(output_tensor.device):
        rc = N.lib().lora_b200_expand(
            output_tensor.data_ptr(), output_tensor.stride(0), inputs.data_ptr(), N.dtype_code(inputs.dtype), T,
            len(slabs), N.ptr_array(slabs), N.int_array(widths), N.int_array(cols), S, r,
            token_lora_mapping.data_ptr(), 1 if add_inputs else 0, N.dtype_code(output_tensor.dtype),
            N.current_stream(output_tensor.device),
        )
    N.check(rc)


@torch.inference_mode()
def lora_shrink(
    inputs: torch.Tensor,
    lora_a_weights: list[torch.Tensor],
    output_tensor: torch.Tensor,
    token_lora_mapping: torch.Tensor,
    token_indices_sorted_by_lora_ids: torch.Tensor,
    num_tokens_per_lora: torch.Tensor,
    lora_token_start_loc: torch.Tensor,
    lora_ids: torch.Tensor,
    no_lora_flag: bool,
    num_active_loras: int,
    scaling: float,
) -> None:
    """``output[s, t] = scaling * inputs[t] @ A_s[slot_t].T``; rows without an adapter are zero.

    The kernel routes by ``token_lora_mapping``; the bucket tensors are accepted for
    signature compatibility (a per-token shrink needs nothing else)."""
    if no_lora_flag:
        return
    shrink_into(output_tensor, inputs, lora_a_weights, token_lora_mapping, scaling)


@torch.inference_mode()
def lora_expand(
    inputs: torch.Tensor,
    lora_b_weights: list[torch.Tensor],
    output_tensor: torch.Tensor,
    token_lora_mapping: torch.Tensor,
    token_indices_sorted_by_lora_ids: torch.Tensor,
    num_tokens_per_lora: torch.Tensor,
    lora_token_start_loc: torch.Tensor,
    lora_ids: torch.Tensor,
    no_lora_flag: bool,
    num_active_loras: int,
    offset_start: int = 0,
    add_inputs: bool = False,
) -> None:
    """``output[t, offset_start + ...] (+)= inputs[s, t] @ B_s[slot_t].T`` for rows with an adapter."""
    if no_lora_flag:
        return
    expand_into(
        output_tensor, inputs, lora_b_weights, token_lora_mapping, offset_start=offset_start, add_inputs=add_inputs
    )


@dataclass
class LoRAKernelMeta:
    """vLLM-style kernel metadata: the ``-1`` bucket is kept with its real token count.

    Buffers are sized ``max_loras + 1`` / ``max_loras + 2`` once and refilled per step,
    unused bucket ids are ``-1`` (``lora_kernel_metadata.py:21-67``).
    """

    token_lora_mapping: torch.Tensor
    token_indices_sorted_by_lora_ids: torch.Tensor
    active_lora_ids: torch.Tensor
    num_tokens_per_lora: torch.Tensor
    lora_token_start_loc: torch.Tensor
    no_lora_flag: bool = False
    num_active_loras: int = 0
    default_num_active_loras: int = 0
    captured_lora_counts: list[int] = field(default_factory=list)

    @staticmethod
    def make(max_loras, max_num_tokens, device, captured_lora_counts=None) -> "LoRAKernelMeta":
        i32 = dict(dtype=torch.int32, device=device)
        return LoRAKernelMeta(
            token_lora_mapping=torch.empty(max_num_tokens, **i32),
            token_indices_sorted_by_lora_ids=torch.empty(max_num_tokens, **i32),
            active_lora_ids=torch.empty(max_loras + 1, **i32),
            num_tokens_per_lora=torch.zeros(max_loras + 1, **i32),
            lora_token_start_loc=torch.zeros(max_loras + 2, **i32),
            default_num_active_loras=max_loras + 1,
            captured_lora_counts=sorted(captured_lora_counts or []),
        )

    def prepare_tensors(self, token_lora_mapping: torch.Tensor) -> None:
        self.active_lora_ids.fill_(-1)
        self.num_tokens_per_lora.zero_()
        self.lora_token_start_loc.zero_()
        self.num_active_loras = 0
        self.no_lora_flag = bool((token_lora_mapping == -1).all().item())
        if self.no_lora_flag:
            return
        n = token_lora_mapping.numel()
        self.token_lora_mapping[:n].copy_(token_lora_mapping, non_blocking=True)
        order = torch.sort(token_lora_mapping, stable=True).indices
        self.token_indices_sorted_by_lora_ids[:n].copy_(order, non_blocking=True)
        ids, counts = torch.unique(token_lora_mapping, sorted=True, return_counts=True)
        k = ids.numel()
        self.active_lora_ids[:k].copy_(ids, non_blocking=True)
        self.num_tokens_per_lora[:k].copy_(counts, non_blocking=True)
        self.lora_token_start_loc[1 : k + 1].copy_(torch.cumsum(counts, dim=0), non_blocking=True)
        if self.captured_lora_counts and k > 0:
            pos = bisect.bisect_left(self.captured_lora_counts, k)
            if pos < len(self.captured_lora_counts):
                k = self.captured_lora_counts[pos]
        self.num_active_loras = k

    def prepare_tensors_on_device(self, token_lora_mapping: torch.Tensor) -> None:
        """:meth:`prepare_tensors` in one kernel launch (``lora_b200_build_metadata``), without sort /
        unique / cumsum launches and without a host read: ``no_lora_flag`` stays False and
        ``num_active_loras`` the buffer capacity, which every kernel of this package accepts (empty and
        ``-1`` buckets exit at once)."""
        from . import _native as N

        n = token_lora_mapping.numel()
        self.token_lora_mapping[:n].copy_(token_lora_mapping, non_blocking=True)
        N.build_metadata(self.token_lora_mapping[:n], self.active_lora_ids.numel() - 1, N.META_KERNEL,
                         self.token_indices_sorted_by_lora_ids, self.active_lora_ids, self.num_tokens_per_lora,
                         self.lora_token_start_loc)
        self.no_lora_flag = False
        self.num_active_loras = self.default_num_active_loras

    def meta_args(self, token_nums: int, specialize_active_lora: bool):
        active = self.num_active_loras if specialize_active_lora else self.default_num_active_loras
        return (
            self.token_lora_mapping[:token_nums],
            self.token_indices_sorted_by_lora_ids[:token_nums],
            self.num_tokens_per_lora,
            self.lora_token_start_loc,
            self.active_lora_ids,
            self.no_lora_flag,
            active,
        )
