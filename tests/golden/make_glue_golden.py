"""Generates tests/golden/glue.npz by running the REFERENCE's modules for the decoder-layer glue on the CPU:
RMSNorm (nanovllm_voxcpm/layers/layernorm.py), SiluAndMul (layers/activation.py, its torch.compile wrapper
switched off so that the plain formula runs) and MiniCPMLongRoPE with its cos / sin cache
(models/voxcpm2/model.py:44-94, model_utils_rope.py), on the seeded inputs of glue_cases.py in fp32 and bf16.

Run where the reference is importable:
    LORA_REFERENCE_ROOT=/path/to/reference python tests/golden/make_glue_golden.py
The model package's __init__ pulls in the audio / server stack; it is registered as a bare package so that
only the model-definition modules execute.
"""

from __future__ import annotations

import os
import sys
import types

os.environ["TORCHDYNAMO_DISABLE"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("LORA_REFERENCE_ROOT") or (sys.argv[1] if len(sys.argv) > 1 else None)
if not REF or not os.path.isdir(REF):
    raise SystemExit("usage: LORA_REFERENCE_ROOT=<checkout of the reference project> python " + os.path.basename(__file__)
                     + "   (or pass the path as the first argument)")
sys.path.insert(0, REF)
sys.path.insert(0, HERE)

for _pkg in ("nanovllm_voxcpm.models", "nanovllm_voxcpm.models.voxcpm2"):
    _m = types.ModuleType(_pkg)
    _m.__path__ = [os.path.join(REF, *_pkg.split("."))]
    sys.modules[_pkg] = _m

import glue_cases as gc  # noqa: E402
from nanovllm_voxcpm.layers.activation import SiluAndMul  # noqa: E402
from nanovllm_voxcpm.layers.layernorm import RMSNorm  # noqa: E402
from nanovllm_voxcpm.models.voxcpm2.model import MiniCPMLongRoPE  # noqa: E402


def as_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().numpy()  # bf16 values are exact in fp32


def main() -> None:
    out = {}
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        d = gc.inputs(dtype)
        norm = RMSNorm(gc.HIDDEN, eps=gc.EPS).to(dtype)
        with torch.no_grad():
            norm.weight.copy_(d["weight"])
            out[f"{tag}/rms"] = as_np(norm(d["x"]))
            normed, hidden = norm(d["x"], d["residual"])
            out[f"{tag}/add_rms"], out[f"{tag}/add_rms_hidden"] = as_np(normed), as_np(hidden)
            layer_hidden = d["residual"] + d["x"]       # the decoder layer's own form
            out[f"{tag}/layer_hidden"], out[f"{tag}/layer_rms"] = as_np(layer_hidden), as_np(norm(layer_hidden))
            out[f"{tag}/silu_mul"] = as_np(SiluAndMul()(d["gate_up"]))
            for name, max_pos in (("short", 128), ("long", gc.MAX_POS)):
                rope = MiniCPMLongRoPE(gc.HEAD_DIM, gc.HEAD_DIM, max_pos, gc.ROPE["base"], gc.ROPE["short_factor"],
                                       gc.ROPE["long_factor"], gc.ROPE["original_max_position"])
                pos = d["positions"] % max_pos
                q, k = rope(pos, d["q"], d["k"])
                out[f"{tag}/rope_{name}_q"], out[f"{tag}/rope_{name}_k"] = as_np(q), as_np(k)
                if tag == "f32":
                    out[f"tables_{name}_cos"], out[f"tables_{name}_sin"] = as_np(rope.cos_cached), as_np(rope.sin_cached)
    np.savez_compressed(os.path.join(HERE, "glue.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
