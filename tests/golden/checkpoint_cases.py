"""Seeded synthetic adapter checkpoints shared by make_checkpoint_golden.py (which feeds them to the
reference's loaders) and tests/test_adapter_checkpoint.py (which feeds them to this package's loader)."""

from __future__ import annotations

import json
import os

import torch
from safetensors.torch import save_file

HIDDEN, KV, INTER, FUSION = 64, 32, 128, 48

# name -> description; "tensors" lists (key, which, out/in dims) in the order they are written
CASES = {
    # every projection of two layers of two backbones, prefixes to drop, a plain linear module, a key to ignore
    "full_fp32": dict(rank=4, alpha=8.0, dtype="float32", config={"r": 4, "alpha": 8.0}, layers=2,
                      projections=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"],
                      prefix="base_model.model.", extra_linear=True, junk_key=True, tp=[1, 2, 4]),
    # q and v only, written v first; bf16 tensors; the alternative config keys
    "qv_bf16": dict(rank=8, alpha=4.0, dtype="bfloat16", config={"rank": 8, "lora_alpha": 4}, layers=1,
                    projections=["v_proj", "q_proj"], prefix="", extra_linear=False, junk_key=False, tp=[1, 2]),
    # rank left out of the config; fp16 tensors; nested prefixes
    "norank_fp16": dict(rank=2, alpha=3.0, dtype="float16", config={"alpha": 3.0}, layers=1,
                        projections=["up_proj", "gate_proj", "down_proj", "o_proj"], prefix="module.model.",
                        extra_linear=True, junk_key=False, tp=[1, 2]),
}

# name -> (tensors as {key: shape}, config json object or raw text)
ERROR_CASES = {
    "no_lora_config_object": ({}, {"alpha": 8}),
    "config_not_object": ({}, [1, 2]),
    "weight_suffix": ({"base_lm.layers.0.self_attn.q_proj.lora_A.weight": (2, 8),
                       "base_lm.layers.0.self_attn.q_proj.lora_B.weight": (8, 2)}, {"lora_config": {"r": 2, "alpha": 8}}),
    "no_alpha": ({"a.q_proj.lora_A": (2, 8), "a.q_proj.lora_B": (8, 2)}, {"lora_config": {"r": 2}}),
    "bad_alpha": ({"a.q_proj.lora_A": (2, 8), "a.q_proj.lora_B": (8, 2)}, {"lora_config": {"r": 2, "alpha": 0}}),
    "no_modules": ({"a.q_proj.weight": (8, 8)}, {"lora_config": {"r": 2, "alpha": 8}}),
    "missing_b": ({"a.q_proj.lora_A": (2, 8), "a.k_proj.lora_A": (2, 8), "a.k_proj.lora_B": (8, 2)},
                  {"lora_config": {"r": 2, "alpha": 8}}),
    "inconsistent_ranks": ({"a.q_proj.lora_A": (2, 8), "a.q_proj.lora_B": (8, 2), "a.o_proj.lora_A": (4, 8),
                            "a.o_proj.lora_B": (8, 4)}, {"lora_config": {"alpha": 8}}),
    "rank_mismatch": ({"a.q_proj.lora_A": (2, 8), "a.q_proj.lora_B": (8, 2)}, {"lora_config": {"r": 4, "alpha": 8}}),
    "bad_rank": ({"a.q_proj.lora_A": (2, 8), "a.q_proj.lora_B": (8, 2)}, {"lora_config": {"r": 0, "alpha": 8}}),
}

_DIMS = {  # projection -> (out, in)
    "q_proj": (HIDDEN, HIDDEN), "k_proj": (KV, HIDDEN), "v_proj": (KV, HIDDEN), "o_proj": (HIDDEN, HIDDEN),
    "gate_proj": (INTER, HIDDEN), "up_proj": (INTER, HIDDEN), "down_proj": (HIDDEN, INTER),
}


def case_tensors(name: str) -> dict[str, torch.Tensor]:
    case = CASES[name]
    gen = torch.Generator().manual_seed(sum(map(ord, name)))
    dtype = getattr(torch, case["dtype"])
    r = case["rank"]
    tensors: dict[str, torch.Tensor] = {}
    for backbone in ("base_lm", "residual_lm"):
        for layer in range(case["layers"]):
            for proj in case["projections"]:
                out_f, in_f = _DIMS[proj]
                block = "self_attn" if proj in ("q_proj", "k_proj", "v_proj", "o_proj") else "mlp"
                key = f"{case['prefix']}{backbone}.layers.{layer}.{block}.{proj}"
                tensors[key + ".lora_A"] = torch.randn(r, in_f, generator=gen).to(dtype)
                tensors[key + ".lora_B"] = torch.randn(out_f, r, generator=gen).to(dtype)
    if case["extra_linear"]:
        tensors["fusion_concat_proj.lora_A"] = torch.randn(r, FUSION, generator=gen).to(dtype)
        tensors["fusion_concat_proj.lora_B"] = torch.randn(FUSION, r, generator=gen).to(dtype)
    if case["junk_key"]:
        tensors["base_lm.layers.0.self_attn.q_proj.weight"] = torch.randn(4, 4, generator=gen).to(dtype)
    return tensors


def write_case(name: str, root: str) -> str:
    path = os.path.join(root, name)
    os.makedirs(path, exist_ok=True)
    save_file(case_tensors(name), os.path.join(path, "lora_weights.safetensors"))
    with open(os.path.join(path, "lora_config.json"), "w", encoding="utf-8") as f:
        json.dump({"lora_config": CASES[name]["config"]}, f)
    return path


def write_error_case(name: str, root: str) -> str:
    shapes, config = ERROR_CASES[name]
    path = os.path.join(root, name)
    os.makedirs(path, exist_ok=True)
    save_file({k: torch.ones(*shape) for k, shape in shapes.items()}, os.path.join(path, "lora_weights.safetensors"))
    with open(os.path.join(path, "lora_config.json"), "w", encoding="utf-8") as f:
        json.dump(config, f)
    return path


def flatten(payload) -> dict[str, torch.Tensor]:
    """A payload (reference's or this package's: same attribute names) as ``{path: tensor}`` plus scalars."""
    out = {"rank": torch.tensor(payload.rank), "alpha": torch.tensor(payload.alpha, dtype=torch.float64),
           "modules": "|".join(payload.modules.keys())}
    for name, m in payload.modules.items():
        out[f"{name}/a"] = m.lora_a
        bs = m.lora_b if isinstance(m.lora_b, list) else [m.lora_b]
        out[f"{name}/nb"] = torch.tensor(len(bs) if isinstance(m.lora_b, list) else 0)
        for i, b in enumerate(bs):
            out[f"{name}/b{i}"] = b
        out[f"{name}/rank"] = torch.tensor(m.effective_rank)
        out[f"{name}/scaling"] = torch.tensor(m.scaling, dtype=torch.float64)
    return out
