"""Decoder-layer glue around the projections as single launches: residual add + RMSNorm, RoPE + KV-cache
store, SiLU * up. Host mirror of the reference's modules for these steps
(``nanovllm_voxcpm/layers/layernorm.py``, ``layers/activation.py``, ``layers/attention.py:10-49``,
``models/voxcpm2/model.py:81-94``); the kernels are ``csrc/glue.cuh`` behind ``lora_b200_glue_*``.
CUDA tensors only, bf16 / fp16; there is no fallback path.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from . import _native as N


def _rows(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with unit column stride")
    return t


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor, eps: float, *,
                 norm_of_rounded_sum: bool = True, out: torch.Tensor | None = None,
                 hidden_out: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor | None]:
    """``hidden = residual + x`` and ``normed = rms_norm(hidden) * weight`` in one pass over the rows.

    Returns ``(normed, hidden)``; ``hidden`` is ``None`` without a residual. ``hidden_out`` may be ``residual``
    itself (in place). ``norm_of_rounded_sum=False`` gives ``RMSNorm.add_rms_forward``'s rounding.
    """
    N.require_cuda(x, residual, weight, out, hidden_out)
    shape = x.shape
    x2 = _rows(x.reshape(-1, shape[-1]), "x")
    T, H = x2.shape
    if weight.numel() != H or weight.dtype != x.dtype:
        raise ValueError("weight must have the row width and the dtype of x")
    normed = out if out is not None else torch.empty(T, H, dtype=x.dtype, device=x.device)
    normed2 = _rows(normed.reshape(-1, H), "out")
    res2 = hid2 = None
    if residual is not None:
        if residual.shape != shape or residual.dtype != x.dtype:
            raise ValueError("residual must match x")
        res2 = _rows(residual.reshape(-1, H), "residual")
        hidden = hidden_out if hidden_out is not None else torch.empty(T, H, dtype=x.dtype, device=x.device)
        hid2 = _rows(hidden.reshape(-1, H), "hidden_out")
    with N.on_device(x.device):
        N.check(N.lib().lora_b200_glue_add_rmsnorm(
            normed2.data_ptr(), normed2.stride(0), N.ptr(hid2), hid2.stride(0) if hid2 is not None else 0,
            x2.data_ptr(), x2.stride(0), N.ptr(res2), res2.stride(0) if res2 is not None else 0, weight.data_ptr(),
            T, H, float(eps), 1 if norm_of_rounded_sum else 0, N.dtype_code(x.dtype), N.current_stream(x.device)))
    return normed2.view(shape), (hid2.view(shape) if hid2 is not None else None)


class RMSNorm(nn.Module):
    """``layers/layernorm.py:6-42``: ``forward(x)`` -> normed; ``forward(x, residual)`` -> (normed, x + residual)."""

    def __init__(self, hidden_size: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.eps = eps
        self.hidden_size = hidden_size
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def rms_forward(self, x: torch.Tensor) -> torch.Tensor:
        return add_rms_norm(x, None, self.weight, self.eps)[0]

    def add_rms_forward(self, x: torch.Tensor, residual: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        return add_rms_norm(x, residual, self.weight, self.eps, norm_of_rounded_sum=False)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        return self.rms_forward(x) if residual is None else self.add_rms_forward(x, residual)


def silu_and_mul(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    N.require_cuda(x, out)
    shape = x.shape
    if shape[-1] % 2:
        raise ValueError("the last dim holds gate | up and must be even")
    inter = shape[-1] // 2
    x2 = _rows(x.reshape(-1, shape[-1]), "x")
    res = out if out is not None else torch.empty(x2.size(0), inter, dtype=x.dtype, device=x.device)
    res2 = _rows(res.reshape(-1, inter), "out")
    with N.on_device(x.device):
        N.check(N.lib().lora_b200_glue_silu_mul(res2.data_ptr(), res2.stride(0), x2.data_ptr(), x2.stride(0), x2.size(0),
                                                inter, N.dtype_code(x.dtype), N.current_stream(x.device)))
    return res2.view(*shape[:-1], inter)


class SiluAndMul(nn.Module):
    """``layers/activation.py:6-14``."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return silu_and_mul(x)


def rope_kv_store(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, *,
                  positions: torch.Tensor | None = None, cos: torch.Tensor | None = None, sin: torch.Tensor | None = None,
                  k_cache: torch.Tensor | None = None, v_cache: torch.Tensor | None = None,
                  slot_mapping: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Rotates q and k of the packed ``qkv [T, (heads + 2 kv_heads) * head_dim]`` rows IN PLACE and stores the
    rotated k and v rows into the paged cache; returns the ``q, k, v`` views ``[T, heads, head_dim]``.

    ``cos`` / ``sin``: ``[max_position, head_dim]`` (the reference's ``cos_cached``) or ``[max_position,
    head_dim / 2]``; ``positions`` int64. Without them nothing is rotated. ``slot_mapping`` int32, -1 = skip;
    the caches are ``[..., kv_heads, head_dim]`` contiguous.
    """
    N.require_cuda(qkv, positions, cos, sin, k_cache, v_cache, slot_mapping)
    qkv2 = _rows(qkv, "qkv")
    T = qkv2.size(0)
    q_size, kv_size = num_heads * head_dim, num_kv_heads * head_dim
    if qkv2.size(1) != q_size + 2 * kv_size:
        raise ValueError("qkv rows must hold q | k | v")
    rope = positions is not None or cos is not None or sin is not None
    table_dim = table_dtype = max_pos = 0
    if rope:
        if positions is None or cos is None or sin is None:
            raise ValueError("rotation needs positions, cos and sin")
        if positions.dtype != torch.int64 or positions.numel() != T or not positions.is_contiguous():
            raise ValueError("positions must be a contiguous int64 tensor with one entry per row")
        if cos.shape != sin.shape or cos.dim() != 2 or cos.dtype != sin.dtype or not (cos.is_contiguous() and sin.is_contiguous()):
            raise ValueError("cos and sin must be contiguous [max_position, dim] tables of one dtype")
        max_pos, table_dim = cos.shape
        table_dtype = N.dtype_code(cos.dtype)
    if (k_cache is None) != (v_cache is None):
        raise ValueError("k_cache and v_cache come together")
    if k_cache is not None:
        if slot_mapping is None or slot_mapping.dtype != torch.int32 or slot_mapping.numel() != T or not slot_mapping.is_contiguous():
            raise ValueError("slot_mapping must be a contiguous int32 tensor with one entry per row")
        for c in (k_cache, v_cache):
            if not c.is_contiguous() or c.dtype != qkv.dtype or c.numel() % kv_size:
                raise ValueError("the caches must be contiguous [..., kv_heads, head_dim] tensors of the dtype of qkv")
    with N.on_device(qkv.device):
        N.check(N.lib().lora_b200_glue_rope_kv_store(
            qkv2.data_ptr(), qkv2.stride(0), T, num_heads, num_kv_heads, head_dim, N.ptr(positions) if rope else None,
            N.ptr(cos) if rope else None, N.ptr(sin) if rope else None, table_dim, table_dtype, max_pos, N.ptr(k_cache),
            N.ptr(v_cache), N.ptr(slot_mapping) if k_cache is not None else None, N.dtype_code(qkv.dtype),
            N.current_stream(qkv.device)))
    q, k, v = qkv2.split([q_size, kv_size, kv_size], dim=-1)
    return (q.view(T, num_heads, head_dim), k.view(T, num_kv_heads, head_dim), v.view(T, num_kv_heads, head_dim))


def store_kvcache(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  slot_mapping: torch.Tensor) -> None:
    """``layers/attention.py:33-49`` for key / value that are the k | v column ranges of one packed qkv buffer is
    what ``rope_kv_store`` does; this form takes separate ``[T, kv_heads, head_dim]`` tensors and copies them."""
    T, heads, dim = key.shape
    packed = torch.empty(T, 2 * heads * dim, dtype=key.dtype, device=key.device)
    packed[:, : heads * dim] = key.reshape(T, -1)
    packed[:, heads * dim:] = value.reshape(T, -1)
    rope_kv_store(packed, 0, heads, dim, k_cache=k_cache, v_cache=v_cache, slot_mapping=slot_mapping)
