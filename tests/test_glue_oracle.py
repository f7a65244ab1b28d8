"""The glue oracle against the reference's own modules (fixtures from tests/golden/make_glue_golden.py)."""

import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
sys.path.insert(0, os.path.dirname(HERE))

import glue_cases as gc  # noqa: E402
from oracle import glue_oracle as GO  # noqa: E402

GOLDEN = np.load(os.path.join(HERE, "golden", "glue.npz"))
BF16_ULP = 2.0 ** -8  # relative spacing of bf16 values: half an ulp of rounding plus the reference's own double roundings


def _close(got: torch.Tensor, key: str, rel: float, abs_: float = 0.0):
    want = torch.from_numpy(GOLDEN[key])
    assert got.shape == want.shape, key
    err = (got.float() - want).abs()
    assert bool((err <= rel * want.abs() + abs_).all()), f"{key}: max err {float(err.max())}"


@pytest.mark.parametrize("tag,dtype", [("f32", torch.float32), ("bf16", torch.bfloat16)])
def test_norms_and_activation(tag, dtype):
    d = gc.inputs(dtype)
    rel = 2e-6 if dtype == torch.float32 else 2 * BF16_ULP
    round_ = (lambda t: t) if dtype == torch.float32 else (lambda t: t.to(dtype))
    _close(round_(GO.rms_norm(d["x"], d["weight"], gc.EPS)), f"{tag}/rms", rel, 1e-6)
    normed, hidden = GO.add_rms_norm(d["x"], d["residual"], d["weight"], gc.EPS, norm_of_rounded_sum=False)
    _close(round_(normed), f"{tag}/add_rms", rel, 1e-6)
    assert torch.equal(hidden.float(), torch.from_numpy(GOLDEN[f"{tag}/add_rms_hidden"]))
    normed, hidden = GO.add_rms_norm(d["x"], d["residual"], d["weight"], gc.EPS, norm_of_rounded_sum=True)
    _close(round_(normed), f"{tag}/layer_rms", rel, 1e-6)
    assert torch.equal(hidden.float(), torch.from_numpy(GOLDEN[f"{tag}/layer_hidden"]))
    _close(round_(GO.silu_and_mul(d["gate_up"])), f"{tag}/silu_mul", rel, 1e-6)


@pytest.mark.parametrize("name,max_pos", [("short", 128), ("long", gc.MAX_POS)])
def test_rope_is_bit_exact(name, max_pos):
    cos, sin = GO.rope_tables(gc.HEAD_DIM, max_pos, gc.ROPE["base"], gc.ROPE["short_factor"], gc.ROPE["long_factor"],
                              gc.ROPE["original_max_position"])
    assert torch.equal(cos, torch.from_numpy(GOLDEN[f"tables_{name}_cos"]))
    assert torch.equal(sin, torch.from_numpy(GOLDEN[f"tables_{name}_sin"]))
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        d = gc.inputs(dtype)
        pos = d["positions"] % max_pos
        for which, heads in (("q", gc.HEADS), ("k", gc.KV_HEADS)):
            got = GO.rope(d[which].view(gc.T, heads, gc.HEAD_DIM), pos, cos, sin).to(dtype).reshape(gc.T, -1)
            assert torch.equal(got.float(), torch.from_numpy(GOLDEN[f"{tag}/rope_{name}_{which}"])), (tag, which)
        # half-width tables give the same rotation
        half = gc.HEAD_DIM // 2
        got = GO.rope(d["q"].view(gc.T, gc.HEADS, gc.HEAD_DIM), pos, cos[:, :half].contiguous(), sin[:, :half].contiguous())
        assert torch.equal(got.to(dtype).reshape(gc.T, -1).float(), torch.from_numpy(GOLDEN[f"{tag}/rope_{name}_q"]))


def test_store_kvcache_skips_minus_one():
    key = torch.arange(3 * 2 * 4, dtype=torch.float32).view(3, 2, 4)
    value = -key
    kc, vc = torch.zeros(2, 4, 2, 4), torch.zeros(2, 4, 2, 4)
    GO.store_kvcache(key, value, kc, vc, torch.tensor([5, -1, 0], dtype=torch.int32))
    assert torch.equal(kc.view(8, 8)[5], key[0].reshape(-1)) and torch.equal(vc.view(8, 8)[0], value[2].reshape(-1))
    assert float(kc.abs().sum()) == float(key[0].abs().sum() + key[2].abs().sum())
