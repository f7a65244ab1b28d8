"""Shared test helpers: tolerance of the path, layer construction from golden cases."""

from __future__ import annotations

import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Tolerance stated for this path: bf16 outputs within max-abs 2e-2 and rel 1e-2 of an
# fp32-accumulated reference.
MAX_ABS = 2e-2
REL = 1e-2


def assert_lora_close(out: torch.Tensor, ref: torch.Tensor, *, max_abs=MAX_ABS, rel=REL, what=""):
    out32, ref32 = out.detach().float().cpu(), ref.detach().float().cpu()
    assert out32.shape == ref32.shape, f"{what}: shape {tuple(out32.shape)} vs {tuple(ref32.shape)}"
    err = (out32 - ref32).abs()
    worst = float(err.max()) if err.numel() else 0.0
    scale = float(ref32.abs().max()) if ref32.numel() else 1.0
    assert worst <= max_abs, f"{what}: max-abs error {worst:.4g} > {max_abs}"
    assert worst <= rel * max(scale, 1.0), f"{what}: relative error {worst / max(scale, 1.0):.4g} > {rel}"


def load_golden(name: str):
    return np.load(os.path.join(GOLDEN, name))


def checksum(*tensors) -> np.ndarray:
    return np.array([float(t.double().sum()) for t in tensors] + [float(t.double().abs().sum()) for t in tensors])


def build_b200_layer(layers_mod, case, inputs, tp_rank, dtype=torch.float32, device="cpu"):
    """Instantiate one of this package's layers for a golden case and load base weights
    and adapter slots (per-rank shards for tp > 1)."""
    import cases

    tp = case.get("tp", 1)
    layers_mod._get_world_size = lambda: tp
    layers_mod._get_rank = lambda: tp_rank
    kind, S, r = case["kind"], case["S"], case["r_max"]
    if kind == "linear":
        layer = layers_mod.LoRALinear(case["in_f"], case["out_f"], bias=case["bias"], max_loras=S, max_lora_rank=r)
        layer.weight.data.copy_(inputs["weights"][0])
        if case["bias"]:
            layer.bias.data.copy_(inputs["bias"])
    elif kind == "row":
        layer = layers_mod.LoRARowParallelLinear(case["in_f"], case["out_f"], bias=case["bias"], max_loras=S, max_lora_rank=r)
        layer.load_base_shard(inputs["weights"][0])
        if case["bias"]:
            layer.bias.data.copy_(inputs["bias"])
    elif kind == "qkv":
        layer = layers_mod.LoRAQKVParallelLinear(
            case["hidden"], case["head"], case["heads"], case["kv_heads"], bias=False, lora_targets=case["targets"],
            max_loras=S, max_lora_rank=r,
        )
        for name, w in zip("qkv", inputs["weights"]):
            layer.load_base_shard(w, name)
    else:
        layer = layers_mod.LoRAMergedColumnParallelLinear(
            case["in_f"], case["outs"], bias=False, lora_targets=case["targets"], max_loras=S, max_lora_rank=r
        )
        for i, w in enumerate(inputs["weights"]):
            layer.load_base_shard(w, i)
    layer = layer.to(device=device, dtype=dtype)
    payload = cases.shard_payload(case, inputs, tp_rank)
    targets = inputs["targets"]
    for slot, ad in payload.items():
        cast = lambda t: t.to(device=device, dtype=dtype)  # noqa: E731
        if kind in ("linear", "row"):
            layer.set_slot_lora(slot, cast(ad["a"][targets[0]]), cast(ad["b"][targets[0]]), ad["rank"], ad["scaling"])
        else:
            layer.set_slot_lora(
                slot, torch.stack([cast(ad["a"][t]) for t in targets]), [cast(ad["b"][t]) for t in targets],
                ad["rank"], ad["scaling"],
            )
    x = inputs["x"]
    if kind == "row" and tp > 1:
        x = x.chunk(tp, 1)[tp_rank]
    return layer, x.to(device=device, dtype=dtype)


class OracleBackend:
    """LoRABackend on the CPU oracle: lets the layers' host logic run without a GPU."""

    def availability(self):
        from nanovllm_voxcpm_b200.lora import LoRAAvailability

        return LoRAAvailability(True, None)

    def shrink(self, x, lora_a):
        return torch.nn.functional.linear(x, lora_a)

    def expand(self, hidden, lora_b, *, scaling):
        return torch.nn.functional.linear(hidden, lora_b) * scaling

    def add_lora(self, y_slices, x, lora_a_slices, lora_b_slices, *, indices, metadata, scaling, y_packed=None):
        from oracle import lora_oracle

        outs = []
        for y, a, b in zip(y_slices, lora_a_slices, lora_b_slices):
            new = lora_oracle.add_lora(y, x, [a], [b], indices, scaling, [0]).to(y.dtype)
            if y_packed is not None or len(y_slices) == 1:
                y.copy_(new)
                outs.append(y)
            else:
                outs.append(new)
        return outs
