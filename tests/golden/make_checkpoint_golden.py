"""Generates tests/golden/checkpoints.npz by running the REFERENCE's adapter-checkpoint loaders
(nanovllm_voxcpm/models/voxcpm2/lora_loader.py and models/voxcpm/lora_loader.py) on the seeded
synthetic checkpoints of checkpoint_cases.py.

Run where the reference is importable:
    LORA_REFERENCE_ROOT=/path/to/reference python tests/golden/make_checkpoint_golden.py
The model packages' __init__ files pull in the audio / server stack, which the loaders do not need;
they are registered as bare packages so that only the loader and model-definition modules execute.
Stored: every payload tensor per case, TP size and rank (both loaders must agree), the module order,
and for the malformed checkpoints the exception type and message.
"""

from __future__ import annotations

import os
import sys
import tempfile
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("LORA_REFERENCE_ROOT") or (sys.argv[1] if len(sys.argv) > 1 else None)
if not REF or not os.path.isdir(REF):
    raise SystemExit("usage: LORA_REFERENCE_ROOT=<checkout of the reference project> python " + os.path.basename(__file__)
                     + "   (or pass the path as the first argument)")
sys.path.insert(0, REF)
sys.path.insert(0, HERE)

for _pkg in ("nanovllm_voxcpm.models", "nanovllm_voxcpm.models.voxcpm2", "nanovllm_voxcpm.models.voxcpm"):
    _m = types.ModuleType(_pkg)
    _m.__path__ = [os.path.join(REF, *_pkg.split("."))]
    sys.modules[_pkg] = _m

import checkpoint_cases as cc  # noqa: E402
from nanovllm_voxcpm.models.voxcpm.lora_loader import load_voxcpm_lora_checkpoint  # noqa: E402
from nanovllm_voxcpm.models.voxcpm2.lora_loader import load_voxcpm2_lora_checkpoint  # noqa: E402


def main() -> None:
    out: dict[str, np.ndarray] = {}
    with tempfile.TemporaryDirectory() as root:
        for name, case in cc.CASES.items():
            path = cc.write_case(name, root)
            for tp in case["tp"]:
                v2 = load_voxcpm2_lora_checkpoint(path, tp_size=tp)
                v1 = load_voxcpm_lora_checkpoint(path, tp_size=tp)
                v2, v1 = (v2 if tp > 1 else [v2]), (v1 if tp > 1 else [v1])
                for r, (p2, p1) in enumerate(zip(v2, v1)):
                    f2, f1 = cc.flatten(p2), cc.flatten(p1)
                    assert f2.keys() == f1.keys() and f2["modules"] == f1["modules"]
                    for k, v in f2.items():
                        if isinstance(v, str):
                            out[f"{name}/tp{tp}/r{r}/{k}"] = np.array(v)
                        else:
                            assert (v == f1[k]).all() and v.dtype == f1[k].dtype, k
                            out[f"{name}/tp{tp}/r{r}/{k}"] = v.numpy()
        for name in cc.ERROR_CASES:
            path = cc.write_error_case(name, root)
            for loader in (load_voxcpm2_lora_checkpoint, load_voxcpm_lora_checkpoint):
                try:
                    loader(path)
                except Exception as exc:  # noqa: BLE001
                    got = f"{type(exc).__name__}: {exc}"
                else:
                    got = "no error"
                assert out.setdefault(f"error/{name}", np.array(got)) == got
    np.savez_compressed(os.path.join(HERE, "checkpoints.npz"), **out)
    print(f"{len(out)} arrays")
    for k in out:
        if k.startswith("error/"):
            print(k, "->", out[k])


if __name__ == "__main__":
    main()
