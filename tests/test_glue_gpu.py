"""Decoder-layer glue kernels (residual add + RMSNorm, RoPE + KV store, SiLU * up) through the C-ABI against the
CPU oracle, the reference-generated fixtures and, at full size, a plain fp32 torch formula on the GPU.

Tolerances: every output is one rounding of an fp32 result, so it may differ from the rounded oracle by one
unit in the last place of the output dtype (relative 2^-8 for bf16, 2^-11 for fp16, written as `ulp` below; the
statistics of the norm add a few 1e-7 relative). The rotation and all copies are bit-exact."""

import os
import sys

import numpy as np
import pytest
import torch

from nanovllm_voxcpm_b200 import glue as G

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
sys.path.insert(0, os.path.dirname(HERE))
import glue_cases as gc  # noqa: E402
from oracle import glue_oracle as GO  # noqa: E402

pytestmark = pytest.mark.gpu
ULP = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}


def _within_one_ulp(got: torch.Tensor, want_f32: torch.Tensor, dtype, what: str):
    err = (got.float().cpu() - want_f32).abs()
    bound = ULP[dtype] * want_f32.abs() * 1.01 + 1e-7
    assert bool((err <= bound).all()), f"{what}: max err {float(err.max())}, worst ratio {float((err / bound).max())}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,H", [(1, 256), (7, 1024), (64, 2048), (300, 4096), (33, 264)])
def test_add_rmsnorm_matches_oracle(dtype, T, H):
    gen = torch.Generator().manual_seed(T * 7 + H)
    x = (torch.randn(T, H, generator=gen) * 1.5).to(dtype)
    res = (torch.randn(T, H, generator=gen) * 3).to(dtype)
    w = (1 + 0.1 * torch.randn(H, generator=gen)).to(dtype)
    xd, rd, wd = x.cuda(), res.cuda(), w.cuda()
    for rounded in (True, False):
        want, want_hidden = GO.add_rms_norm(x, res, w, 1e-6, rounded)
        normed, hidden = G.add_rms_norm(xd, rd, wd, 1e-6, norm_of_rounded_sum=rounded)
        assert torch.equal(hidden.cpu(), want_hidden)
        _within_one_ulp(normed, want, dtype, f"normed rounded={rounded}")
    # no residual; strided input rows; output into a column range of a wider buffer
    wide = torch.zeros(T, 2 * H + 8, dtype=dtype, device="cuda")
    wide[:, 8:8 + H] = xd
    out = torch.full((T, H + 16), 7.0, dtype=dtype, device="cuda")
    normed, hidden = G.add_rms_norm(wide[:, 8:8 + H], None, wd, 1e-6, out=out[:, :H])
    assert hidden is None and bool((out[:, H:] == 7).all())
    _within_one_ulp(out[:, :H], GO.rms_norm(x, w, 1e-6), dtype, "plain rms_norm")
    # in place: the sum replaces the residual
    normed, hidden = G.add_rms_norm(xd, rd, wd, 1e-6, hidden_out=rd)
    assert hidden.data_ptr() == rd.data_ptr() and torch.equal(rd.cpu(), GO.add_rms_norm(x, res, w, 1e-6, True)[1])
    # the module form of the reference
    m = G.RMSNorm(H).to("cuda", dtype)
    with torch.no_grad():
        m.weight.copy_(wd)
    _within_one_ulp(m(xd), GO.rms_norm(x, w, 1e-6), dtype, "RMSNorm(x)")
    normed, new_res = m(xd, res.cuda())
    _within_one_ulp(normed, GO.add_rms_norm(x, res, w, 1e-6, False)[0], dtype, "RMSNorm(x, residual)")
    assert torch.equal(new_res.cpu(), (x.float() + res.float()).to(dtype))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,I", [(1, 64), (9, 1024), (256, 4096), (37, 520)])
def test_silu_mul_matches_oracle(dtype, T, I):
    gen = torch.Generator().manual_seed(T + I)
    x = (torch.randn(T, 2 * I, generator=gen) * 3).to(dtype)
    got = G.silu_and_mul(x.cuda())
    assert got.shape == (T, I)
    _within_one_ulp(got, GO.silu_and_mul(x), dtype, "silu_mul")
    wide = torch.zeros(T, 2 * I + 16, dtype=dtype, device="cuda")
    wide[:, 16:] = x.cuda()
    out = torch.zeros(T, I + 8, dtype=dtype, device="cuda")
    G.silu_and_mul(wide[:, 16:], out=out[:, :I])
    assert torch.equal(out[:, :I], got) and bool((out[:, I:] == 0).all())
    assert torch.equal(G.SiluAndMul()(x.cuda().view(1, T, 2 * I)), got.view(1, T, I))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("heads,kv_heads,dim,table", [(16, 2, 64, "full_f32"), (4, 4, 128, "half_f32"), (8, 1, 64, "full_bf16"),
                                                      (2, 2, 32, "half_bf16")])
def test_rope_kv_store_is_bit_exact(dtype, heads, kv_heads, dim, table):
    T, max_pos, slots = 50, 300, 128
    gen = torch.Generator().manual_seed(heads * dim)
    qkv = torch.randn(T, (heads + 2 * kv_heads) * dim, generator=gen).to(dtype)
    positions = torch.randint(0, max_pos, (T,), generator=gen)
    cos, sin = GO.rope_tables(dim, max_pos, 10000.0)
    if table.startswith("half"):
        cos, sin = cos[:, : dim // 2].contiguous(), sin[:, : dim // 2].contiguous()
    if table.endswith("bf16"):
        cos, sin = cos.bfloat16(), sin.bfloat16()
    slot_mapping = torch.randperm(slots, generator=gen)[:T].to(torch.int32)
    slot_mapping[::7] = -1
    k_cache = torch.full((slots // 16, 16, kv_heads, dim), 3.0, dtype=dtype)
    v_cache = torch.full_like(k_cache, -3.0)
    q0, k0, v0 = qkv.split([heads * dim, kv_heads * dim, kv_heads * dim], dim=-1)
    want_q = GO.rope(q0.reshape(T, heads, dim), positions, cos, sin).to(dtype)
    want_k = GO.rope(k0.reshape(T, kv_heads, dim), positions, cos, sin).to(dtype)
    want_kc, want_vc = k_cache.clone(), v_cache.clone()
    GO.store_kvcache(want_k, v0.reshape(T, kv_heads, dim), want_kc, want_vc, slot_mapping)

    # the packed rows sit inside a wider buffer (row pitch != row width)
    buf = torch.zeros(T, qkv.size(1) + 24, dtype=dtype, device="cuda")
    buf[:, : qkv.size(1)] = qkv.cuda()
    kc, vc = k_cache.cuda(), v_cache.cuda()
    q, k, v = G.rope_kv_store(buf[:, : qkv.size(1)], heads, kv_heads, dim, positions=positions.cuda(), cos=cos.cuda(),
                              sin=sin.cuda(), k_cache=kc, v_cache=vc, slot_mapping=slot_mapping.cuda())
    assert torch.equal(q.cpu(), want_q) and torch.equal(k.cpu(), want_k)
    assert torch.equal(v.cpu(), v0.reshape(T, kv_heads, dim)) and bool((buf[:, qkv.size(1):] == 0).all())
    assert torch.equal(kc.cpu(), want_kc) and torch.equal(vc.cpu(), want_vc)

    # no rotation (use_rope = False) still stores; no cache still rotates
    kc2, vc2 = k_cache.cuda(), v_cache.cuda()
    raw = qkv.cuda()
    G.rope_kv_store(raw, heads, kv_heads, dim, k_cache=kc2, v_cache=vc2, slot_mapping=slot_mapping.cuda())
    want_kc2, want_vc2 = k_cache.clone(), v_cache.clone()
    GO.store_kvcache(k0.reshape(T, kv_heads, dim), v0.reshape(T, kv_heads, dim), want_kc2, want_vc2, slot_mapping)
    assert torch.equal(raw.cpu(), qkv) and torch.equal(kc2.cpu(), want_kc2) and torch.equal(vc2.cpu(), want_vc2)
    raw2 = qkv.cuda()
    q2, k2, _ = G.rope_kv_store(raw2, heads, kv_heads, dim, positions=positions.cuda(), cos=cos.cuda(), sin=sin.cuda())
    assert torch.equal(q2.cpu(), want_q) and torch.equal(k2.cpu(), want_k)
    kc3, vc3 = k_cache.cuda(), v_cache.cuda()
    G.store_kvcache(want_k.cuda(), v0.reshape(T, kv_heads, dim).cuda(), kc3, vc3, slot_mapping.cuda())
    assert torch.equal(kc3.cpu(), want_kc) and torch.equal(vc3.cpu(), want_vc)


def test_reference_fixtures():
    """bf16 outputs of the reference's own modules (CPU): rotation bit-exact, the rest within the reference's own
    double roundings (two units in the last place)."""
    golden = np.load(os.path.join(HERE, "golden", "glue.npz"))
    d = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in gc.inputs(torch.bfloat16).items()}

    def close(got, key):
        want = torch.from_numpy(golden[key])
        err = (got.float().cpu() - want).abs()
        assert bool((err <= 2 * ULP[torch.bfloat16] * want.abs() + 1e-6).all()), key

    close(G.add_rms_norm(d["x"], None, d["weight"], gc.EPS)[0], "bf16/rms")
    normed, hidden = G.add_rms_norm(d["x"], d["residual"], d["weight"], gc.EPS, norm_of_rounded_sum=False)
    close(normed, "bf16/add_rms")
    assert torch.equal(hidden.float().cpu(), torch.from_numpy(golden["bf16/add_rms_hidden"]))
    normed, hidden = G.add_rms_norm(d["x"], d["residual"], d["weight"], gc.EPS)
    close(normed, "bf16/layer_rms")
    assert torch.equal(hidden.float().cpu(), torch.from_numpy(golden["bf16/layer_hidden"]))
    close(G.silu_and_mul(d["gate_up"]), "bf16/silu_mul")
    for name, max_pos in (("short", 128), ("long", gc.MAX_POS)):
        cos, sin = (torch.from_numpy(golden[f"tables_{name}_{t}"]).cuda() for t in ("cos", "sin"))
        qkv = torch.cat((d["q"], d["k"], d["k"]), dim=-1).contiguous()
        q, k, _ = G.rope_kv_store(qkv, gc.HEADS, gc.KV_HEADS, gc.HEAD_DIM, positions=(d["positions"] % max_pos), cos=cos, sin=sin)
        assert torch.equal(q.reshape(gc.T, -1).float().cpu(), torch.from_numpy(golden[f"bf16/rope_{name}_q"]))
        assert torch.equal(k.reshape(gc.T, -1).float().cpu(), torch.from_numpy(golden[f"bf16/rope_{name}_k"]))


def test_full_size_against_torch_fp32():
    """Prefill-sized batch (8192 rows) against the fp32 formulas evaluated by torch on the GPU."""
    T, H, I, heads, kv_heads, dim = 8192, 1024, 4096, 16, 2, 64
    dtype = torch.bfloat16
    gen = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(T, H, device="cuda", generator=gen).to(dtype)
    res = torch.randn(T, H, device="cuda", generator=gen).to(dtype)
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=gen)).to(dtype)
    normed, hidden = G.add_rms_norm(x, res, w, 1e-6)
    assert torch.equal(hidden, (x.float() + res.float()).to(dtype))
    want = GO.rms_norm(hidden, w, 1e-6)  # torch ops: run on the GPU for GPU tensors
    assert bool(((normed.float() - want).abs() <= ULP[dtype] * 1.01 * want.abs() + 1e-7).all())
    gu = (torch.randn(T, 2 * I, device="cuda", generator=gen) * 2).to(dtype)
    got, want = G.silu_and_mul(gu), GO.silu_and_mul(gu)
    assert bool(((got.float() - want).abs() <= ULP[dtype] * 1.01 * want.abs() + 1e-7).all())
    qkv = torch.randn(T, (heads + 2 * kv_heads) * dim, device="cuda", generator=gen).to(dtype)
    pos = torch.randint(0, 4096, (T,), device="cuda", generator=gen)
    cos, sin = (t.cuda() for t in GO.rope_tables(dim, 4096, 10000.0))
    slot = torch.randperm(T * 2, device="cuda", generator=gen)[:T].to(torch.int32)
    kc = torch.zeros(T * 2 // 256, 256, kv_heads, dim, dtype=dtype, device="cuda")
    vc = torch.zeros_like(kc)
    q0, k0, v0 = (t.clone() for t in qkv.split([heads * dim, kv_heads * dim, kv_heads * dim], dim=-1))
    q, k, v = G.rope_kv_store(qkv, heads, kv_heads, dim, positions=pos, cos=cos, sin=sin, k_cache=kc, v_cache=vc, slot_mapping=slot)
    assert torch.equal(q, GO.rope(q0.view(T, heads, dim), pos, cos, sin).to(dtype))
    want_k = GO.rope(k0.view(T, kv_heads, dim), pos, cos, sin).to(dtype)
    assert torch.equal(k, want_k)
    assert torch.equal(kc.view(-1, kv_heads, dim)[slot.long()], want_k) and torch.equal(vc.view(-1, kv_heads, dim)[slot.long()], v0.view(T, kv_heads, dim))


def test_bad_arguments():
    x = torch.zeros(4, 260, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 8"):
        G.add_rms_norm(x, None, torch.ones(260, dtype=torch.bfloat16, device="cuda"), 1e-6)
    with pytest.raises(RuntimeError, match="bf16 and fp16"):
        G.silu_and_mul(torch.zeros(4, 64, device="cuda"))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        G.silu_and_mul(torch.zeros(4, 64, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="positions, cos and sin"):
        G.rope_kv_store(torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda"), 2, 1, 64,
                        positions=torch.zeros(4, dtype=torch.int64, device="cuda"))
