"""Parity of the CUDA path (through the C-ABI) against the CPU oracle on identical
seeded inputs, against the reference-generated fixtures and the reference tests'
known answers.  Tolerance of the path: bf16 outputs within max-abs 2e-2 and rel 1e-2 of
the fp32-accumulated oracle; rows without an adapter must keep their exact bits."""

import numpy as np
import pytest
import torch

import cases
from helpers import assert_lora_close, build_b200_layer, load_golden
from nanovllm_voxcpm_b200 import _native as N
from nanovllm_voxcpm_b200 import batch_plan as BP
from nanovllm_voxcpm_b200 import context as CTX
from nanovllm_voxcpm_b200 import layers as L
from nanovllm_voxcpm_b200 import lora as LORA
from nanovllm_voxcpm_b200 import workloads as W
from nanovllm_voxcpm_b200.lora_ops import LoRAKernelMeta, lora_expand, lora_shrink
from oracle import lora_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _clean():
    LORA.set_backend_for_testing(None)
    CTX.reset_lora_context()
    yield
    N.set_option(N.OPT_CLUSTER, 0)
    N.set_option(N.OPT_PDL, 1)
    N.set_option(N.OPT_KSPLIT, 1)
    CTX.reset_lora_context()
    assert N.device_status() == 0, "a kernel gave up a bounded wait"


def metadata_for(slots: torch.Tensor, convention: str, S: int) -> LORA.LoRAMetadata:
    """The three index conventions of the reference, built on the device."""
    slots_cpu = slots.cpu()
    if convention == "eager":
        ctx = BP.build_lora_context_from_batch_plan(
            BP.build_lora_batch_plan_from_token_to_slot({}, slots_cpu.tolist()), device=DEV
        )
    elif convention == "graph":
        bufs = BP.GraphLoRABuffers.make(slots_cpu.numel() + 5, S, device=DEV)
        bufs.load_plan(BP.build_lora_batch_plan_from_token_to_slot({}, slots_cpu.tolist()))
        ctx = bufs.context(slots_cpu.numel())
    elif convention == "vllm":
        km = LoRAKernelMeta.make(S, slots_cpu.numel(), DEV)
        km.prepare_tensors(slots_cpu.to(DEV))
        tts, srt, cnt, off, ids, flag, n = km.meta_args(slots_cpu.numel(), specialize_active_lora=False)
        return LORA.LoRAMetadata(tts, srt, ids, cnt, off, flag, n)
    else:
        raise AssertionError(convention)
    return LORA.LoRAMetadata(ctx.token_to_slot, ctx.token_indices_sorted_by_slot, ctx.active_slot_ids,
                             ctx.num_tokens_per_slot, ctx.slot_start_offsets, ctx.no_lora_flag, ctx.num_active_loras)


def run_add(p: W.Projection, impl: int, convention: str = "eager", *, use_ranks=False, scaling=1.0,
            scale_per_slot=None, y_pad=0, x_pad=0):
    """One lora_b200_add launch on device copies of ``p``; returns (y_out, y_in) on the CPU."""
    d = p.to_device(DEV)
    S = d.a_slabs[0].shape[0]
    if y_pad or x_pad:  # row-strided views into wider buffers
        ybuf = torch.zeros(d.y.shape[0], d.y.shape[1] + y_pad, dtype=d.y.dtype, device=DEV)
        xbuf = torch.zeros(d.x.shape[0], d.x.shape[1] + x_pad, dtype=d.x.dtype, device=DEV)
        ybuf[:, : d.y.shape[1]] = d.y
        xbuf[:, : d.x.shape[1]] = d.x
        y, x = ybuf[:, : d.y.shape[1]], xbuf[:, : d.x.shape[1]]
    else:
        y, x = d.y.clone(), d.x
    meta = metadata_for(d.token_to_slot, convention, S)
    LORA.launch_add(y, x, d.a_slabs, d.b_slabs, d.out_sizes, d.col_offsets, meta, scaling,
                    rank_per_slot=d.ranks if use_ranks else None,
                    scale_per_slot=None if scale_per_slot is None else scale_per_slot.to(DEV), impl=impl)
    torch.cuda.synchronize()
    return y.cpu(), p.y


def check_against_oracle(p, out, y_in, scaling=1.0, scale_per_slot=None, what=""):
    ref = O.add_lora(y_in, p.x, p.a_slabs, p.b_slabs, p.token_to_slot, scaling, p.col_offsets, scale_per_slot)
    assert_lora_close(out, ref, what=what)
    none = p.token_to_slot < 0
    assert torch.equal(out[none].view(torch.int16), y_in[none].view(torch.int16)), f"{what}: rows without adapter changed"
    touched = (out[~none].float() - y_in[~none].float()).abs().max() if (~none).any() else torch.tensor(1.0)
    assert float(touched) > 0, f"{what}: no delta was applied"


# ------------------------------------------------------------------ decode BGMV
@pytest.mark.parametrize("convention", ["eager", "graph", "vllm"])
@pytest.mark.parametrize("impl", [N.IMPL_GENERIC, N.IMPL_BGMV], ids=["generic", "bgmv"])
@pytest.mark.parametrize("name", ["qkv", "o", "gate_up", "down"])
def test_decode_projection_matches_oracle(name, impl, convention):
    p = W.decode_projection(name, seed=7)
    out, y_in = run_add(p, impl, convention)
    check_against_oracle(p, out, y_in, what=f"{name}/{convention}")
    out2, _ = run_add(p, impl, convention)
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16)), "two runs differ bitwise"


@pytest.mark.parametrize("cluster", [1, 2, 4, 8])
@pytest.mark.parametrize("pdl", [0, 1])
def test_bgmv_cluster_sizes(cluster, pdl):
    N.set_option(N.OPT_CLUSTER, cluster)
    N.set_option(N.OPT_PDL, pdl)
    for name in ("qkv", "down"):
        p = W.decode_projection(name, seed=3, T=96, S=8)
        out, y_in = run_add(p, N.IMPL_BGMV, "graph")
        check_against_oracle(p, out, y_in, what=f"{name}/C{cluster}/pdl{pdl}")


def test_bgmv_many_tokens_per_slot_and_single_token():
    # 200 rows on 2 slots: up to 7 passes of 16 tokens per bucket; then a 1-row batch
    p = W.make_projection(5, 200, 1024, [1024, 128, 128], 2, 32, p_none=0.2)
    out, y_in = run_add(p, N.IMPL_BGMV)
    check_against_oracle(p, out, y_in, what="many tokens")
    p1 = W.make_projection(6, 1, 1024, [1024], 4, 32, token_to_slot=[3])
    out, y_in = run_add(p1, N.IMPL_BGMV)
    check_against_oracle(p1, out, y_in, what="one token")


@pytest.mark.parametrize("ksplit", [1, 0])
def test_bgmv_long_input_rows(ksplit):
    """Input rows of 4 or more K parts of 1024 columns: the K parts are dealt over the cluster and fp32
    partial sums are exchanged (or, switched off, every CTA walks all K parts of its rank rows)."""
    N.set_option(N.OPT_KSPLIT, ksplit)
    try:
        # 3 slots x about 36 rows: three passes of 16 tokens (receive buffers alternate); 5 K parts on 4 CTAs
        p = W.make_projection(15, 120, 4096, [1024], 3, 32, p_none=0.1)
        out, y_in = run_add(p, N.IMPL_BGMV, "graph")
        check_against_oracle(p, out, y_in, what=f"in 4096 / ksplit {ksplit}")
        p = W.make_projection(16, 50, 5120, [512, 256], 5, 32, p_none=0.1)
        out, y_in = run_add(p, N.IMPL_BGMV)
        check_against_oracle(p, out, y_in, what=f"in 5120 / ksplit {ksplit}")
        # ragged last K part (512 of 1024 columns), per-slot ranks and scales, overwrite form
        sps = torch.tensor([1.0, 0.5, 2.0, 1.5])
        p = W.make_projection(17, 40, 4608, [768], 4, 64, ranks=[64, 16, 32, 8])
        out, y_in = run_add(p, N.IMPL_BGMV, use_ranks=True, scaling=0.5, scale_per_slot=sps, x_pad=8)
        check_against_oracle(p, out, y_in, 0.5, sps, what=f"in 4608 / ksplit {ksplit}")
    finally:
        N.set_option(N.OPT_KSPLIT, 1)


def test_bgmv_mixed_ranks_scales_and_strides():
    ranks = [(8, 16, 64)[s % 3] for s in range(6)]
    p = W.make_projection(9, 70, 2048, [2048, 256, 256], 6, 64, ranks=ranks, p_none=0.15)
    sps = torch.tensor([1.0, 0.5, 2.0, 1.5, 0.25, 1.0])
    for use_ranks in (False, True):
        out, y_in = run_add(p, N.IMPL_BGMV, "graph", use_ranks=use_ranks, scaling=0.5, scale_per_slot=sps,
                            y_pad=24, x_pad=8)
        check_against_oracle(p, out, y_in, 0.5, sps, what=f"ranks={use_ranks}")
    # per-slot rank 0 = empty slot: exact zero delta for its rows
    p.ranks[2] = 0
    p.a_slabs = [a.clone() for a in p.a_slabs]
    p.b_slabs = [b.clone() for b in p.b_slabs]
    for a, b in zip(p.a_slabs, p.b_slabs):
        a[2].zero_()
        b[2].zero_()
    out, y_in = run_add(p, N.IMPL_BGMV, use_ranks=True)
    rows = p.token_to_slot == 2
    assert rows.any() and torch.equal(out[rows], y_in[rows])
    check_against_oracle(p, out, y_in, what="empty slot")


def test_zero_width_slice_and_auto_dispatch():
    p = W.make_projection(4, 40, 1024, [512, 0, 256], 4, 32)
    p.a_slabs[1] = p.a_slabs[0]  # never read
    for impl in (N.IMPL_AUTO, N.IMPL_GENERIC, N.IMPL_BGMV):
        out, y_in = run_add(p, impl)
        check_against_oracle(p, out, y_in, what=f"impl {impl}")


def test_unsupported_shapes_are_reported_not_launched():
    p = W.make_projection(4, 8, 1000, [64], 2, 16)  # in % 32 != 0, r % 32 != 0
    with pytest.raises(RuntimeError, match="fused decode kernel"):
        run_add(p, N.IMPL_BGMV)
    out, y_in = run_add(p, N.IMPL_AUTO)  # auto falls back to the generic kernel
    check_against_oracle(p, out, y_in, what="auto->generic")


# --------------------------------------------------------------- config 1 / dtypes
def test_config1_matches_reference_fixture():
    g = load_golden("config1.npz")
    p = W.config1(0)
    out, y_in = run_add(p, N.IMPL_AUTO)
    assert_lora_close(out, torch.from_numpy(g["y"]), what="config1 vs reference fixture")
    check_against_oracle(p, out, y_in, what="config1")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.float16, 2e-2)])
def test_generic_kernel_other_dtypes(dtype, tol):
    p = W.make_projection(21, 33, 160, [48, 24], 3, 8, dtype=dtype, p_none=0.3)
    d = p.to_device(DEV)
    y = d.y.clone()
    LORA.launch_add(y, d.x, d.a_slabs, d.b_slabs, d.out_sizes, d.col_offsets,
                    metadata_for(d.token_to_slot, "eager", 3), 0.5, impl=N.IMPL_AUTO)
    ref = O.add_lora(p.y, p.x, p.a_slabs, p.b_slabs, p.token_to_slot, 0.5, p.col_offsets)
    assert_lora_close(y, ref, max_abs=tol, what=str(dtype))
    none = p.token_to_slot < 0
    assert torch.equal(y.cpu()[none], p.y[none])


def test_shrink_and_expand_ops_match_oracle():
    """Raw ops with the reference's positional signature and vLLM-style metadata
    (tests/unit/test_lora_cuda.py:836-911)."""
    dtype = torch.float16
    g = torch.Generator().manual_seed(2)
    x = (torch.arange(4 * 160, dtype=torch.float32).reshape(4, 160) / 100).to(dtype)
    a = torch.randn(2, 8, 160, generator=g).to(dtype)
    slots = torch.tensor([0, 1, 0, 1], dtype=torch.int32)
    meta = (slots.to(DEV), torch.tensor([0, 2, 1, 3], dtype=torch.int32, device=DEV),
            torch.tensor([2, 2, 0], dtype=torch.int32, device=DEV), torch.tensor([0, 2, 4, 4], dtype=torch.int32, device=DEV),
            torch.tensor([0, 1, -1], dtype=torch.int32, device=DEV), False, 2)
    out = torch.empty((1, 4, 8), device=DEV, dtype=dtype)
    lora_shrink(x.to(DEV), [a.to(DEV)], out, *meta, 0.5)
    assert_lora_close(out, O.shrink(x, [a], slots, 0.5), max_abs=5e-2, rel=5e-2)

    # the reference's split-K shape (tests/unit/test_lora_cuda.py:875-911): K = 4096, rank 1, same metadata; its own
    # bound is 2e-1 (bf16 atomics over the K splits), here the sum is kept in fp32 and rounded once
    x = torch.randn(4, 4096, generator=g).to(dtype)
    a = torch.randn(2, 1, 4096, generator=g).to(dtype)
    out = torch.empty((1, 4, 1), device=DEV, dtype=dtype)
    lora_shrink(x.to(DEV), [a.to(DEV)], out, *meta, 0.5)
    want = O.shrink(x, [a], slots, 0.5)
    torch.testing.assert_close(out.float().cpu(), want, atol=5e-2, rtol=1e-2)

    # bf16, two slices, fp32 intermediate (the row-parallel [T, r] exchange format)
    p = W.make_projection(31, 50, 256, [64, 32], 4, 16, p_none=0.2)
    d = p.to_device(DEV)
    meta = (d.token_to_slot, None, None, None, None, False, 0)
    tmp32 = torch.empty((2, 50, 16), device=DEV, dtype=torch.float32)
    lora_shrink(d.x, d.a_slabs, tmp32, *meta, 1.0)
    ref_tmp = O.shrink(p.x, p.a_slabs, p.token_to_slot)
    torch.testing.assert_close(tmp32.cpu(), ref_tmp, atol=1e-4, rtol=1e-4)
    assert not tmp32.cpu()[:, p.token_to_slot < 0].any()  # zero rows without adapter
    y = d.y.clone()
    lora_expand(tmp32, d.b_slabs, y, *meta, offset_start=0, add_inputs=True)
    assert_lora_close(y, O.expand(p.y, ref_tmp, p.b_slabs, p.token_to_slot))
    y2 = torch.zeros_like(d.y)
    lora_expand(tmp32[1:].contiguous(), d.b_slabs[1:], y2, *meta, offset_start=64, add_inputs=False)
    ref2 = O.expand(torch.zeros_like(p.y), ref_tmp[1:], p.b_slabs[1:], p.token_to_slot, 64, False)
    assert_lora_close(y2, ref2)
    assert not y2.cpu()[:, :64].any()


@pytest.mark.parametrize("name", ["qkv", "o", "gate_up", "down"])
def test_shrink_and_expand_ops_full_size_prefill(name):
    """``lora_shrink`` / ``lora_expand`` on the prefill configuration at full size (bf16 intermediate, 8172 rows):
    these sizes take the tensor-core kernels; compared with the oracle's two halves, rows without adapter zero
    in the intermediate and bit-exact in the output."""
    p = W.prefill_projection(name, seed=0)
    p.token_to_slot[700:777] = -1
    d = p.to_device(DEV)
    n, T, r = len(p.a_slabs), p.x.shape[0], p.a_slabs[0].shape[1]
    meta = (d.token_to_slot, None, None, None, None, False, 0)
    tmp = torch.full((n, T, r), 7.0, device=DEV, dtype=torch.bfloat16)
    lora_shrink(d.x, d.a_slabs, tmp, *meta, 0.5)
    torch.cuda.synchronize()
    ref_tmp = O.shrink(p.x, p.a_slabs, p.token_to_slot, 0.5)
    assert_lora_close(tmp, ref_tmp, what=f"shrink / {name}")
    none = p.token_to_slot < 0
    assert not tmp.cpu()[:, none].any(), "rows without adapter are not zero in the intermediate"
    # expand from the oracle's intermediate rounded to bf16 (so that only the expand is under test); the last
    # slices at a column offset, as a tensor-parallel shard's call has them
    tmp_in = ref_tmp.to(torch.bfloat16)
    want = O.expand(p.y, tmp_in.float(), p.b_slabs, p.token_to_slot)
    y = d.y.clone()
    lora_expand(tmp_in.to(DEV), d.b_slabs, y, *meta, offset_start=0, add_inputs=True)
    torch.cuda.synchronize()
    assert_lora_close(y, want, what=f"expand / {name}")
    assert torch.equal(y.cpu()[none].view(torch.int16), p.y[none].view(torch.int16)), "rows without adapter changed"
    k = len(p.b_slabs) - 1
    y2 = d.y.clone()
    lora_expand(tmp_in[k:].contiguous().to(DEV), d.b_slabs[k:], y2, *meta, offset_start=p.col_offsets[k], add_inputs=True)
    torch.cuda.synchronize()
    want2 = O.expand(p.y, tmp_in[k:].float(), p.b_slabs[k:], p.token_to_slot, p.col_offsets[k], True)
    assert_lora_close(y2, want2, what=f"expand at an offset / {name}")
    assert N.device_status(reset=True) == 0


# ------------------------------------------------------ backend protocol / layers
def test_backend_add_lora_contract():
    """tests/unit/test_lora_cuda.py:804-833 (fp16, scaling 0.5 -> [4, 10]) and the
    in-place / fresh-buffer rules of lora.py:276-289."""
    be = LORA.B200LoRABackend()
    assert be.availability().available
    y = torch.zeros(2, 1, device=DEV, dtype=torch.float16)
    x = torch.tensor([[2.0, 3.0], [5.0, 7.0]], device=DEV, dtype=torch.float16)
    meta = LORA.LoRAMetadata(torch.zeros(2, dtype=torch.int32, device=DEV), torch.arange(2, dtype=torch.int32, device=DEV),
                             torch.tensor([0], dtype=torch.int32, device=DEV), torch.tensor([2], dtype=torch.int32, device=DEV),
                             torch.tensor([0, 2], dtype=torch.int32, device=DEV), False, 1)
    out = be.add_lora([y], x, [torch.tensor([[[1.0, 0.0]]], device=DEV, dtype=torch.float16)],
                      [torch.tensor([[[4.0]]], device=DEV, dtype=torch.float16)],
                      indices=torch.zeros(2, dtype=torch.long, device=DEV), metadata=meta, scaling=0.5)[0]
    assert out.data_ptr() == y.data_ptr() and out.cpu().flatten().tolist() == [4.0, 10.0]

    p = W.make_projection(8, 24, 1024, [256, 128], 4, 32).to_device(DEV)
    m = metadata_for(p.token_to_slot, "eager", 4)
    parts = list(p.y.split(p.out_sizes, dim=-1))
    before = p.y.clone()
    fresh = be.add_lora(parts, p.x, p.a_slabs, p.b_slabs, indices=p.token_to_slot, metadata=m, scaling=1.0)
    assert torch.equal(p.y, before), "inputs must stay untouched without y_packed"
    packed = p.y.clone()
    same = be.add_lora(list(packed.split(p.out_sizes, dim=-1)), p.x, p.a_slabs, p.b_slabs, indices=p.token_to_slot,
                       metadata=m, scaling=1.0, y_packed=packed)
    assert same[0].data_ptr() == packed.data_ptr()
    assert torch.equal(torch.cat(fresh, -1), packed)
    ref = O.add_lora(before, p.x, p.a_slabs, p.b_slabs, p.token_to_slot.cpu())
    assert_lora_close(packed, ref)
    # single-adapter helpers of the protocol
    a1, b1 = p.a_slabs[0][1], p.b_slabs[0][1]
    h = be.shrink(p.x, a1)
    assert_lora_close(h, p.x.float().cpu() @ a1.float().cpu().T)
    e = be.expand(h, b1, scaling=0.5)
    assert_lora_close(e, (h.float().cpu() @ b1.float().cpu().T) * 0.5)


@pytest.mark.parametrize("case", cases.LAYER_CASES, ids=lambda c: c["name"])
def test_layers_match_reference_fixture_fp32(case):
    g = load_golden("layers.npz")
    inputs = cases.build_inputs(case)
    saved = L.dist.all_reduce
    L.dist.all_reduce = lambda t, *a, **k: t
    try:
        for rank in range(case.get("tp", 1)):
            layer, x = build_b200_layer(L, case, inputs, rank, dtype=torch.float32, device=DEV)
            CTX.set_lora_context(CTX.build_lora_context_from_token_to_slot(inputs["slots"].to(DEV)))
            with torch.no_grad():
                y = layer(x)
            torch.testing.assert_close(y.cpu(), torch.from_numpy(g[f"{case['name']}/y_rank{rank}"]), atol=2e-4, rtol=1e-4)
            CTX.reset_lora_context()
            with torch.no_grad():
                base = layer(x)
            none = inputs["slots"] < 0
            assert torch.equal(y.cpu()[none], base.cpu()[none])
    finally:
        L.dist.all_reduce = saved
        L._get_world_size = lambda: 1
        L._get_rank = lambda: 0


def test_kat_layers_on_device():
    """tests/unit/test_lora_cuda.py:135-189 and :576-615 through this package's layers."""
    layer = L.LoRALinear(3, 2, bias=False, max_loras=2, max_lora_rank=4).to(DEV)
    layer.weight.data.zero_()
    layer.set_slot_lora(0, torch.tensor([[1.0, 0, 0], [0, 1.0, 0]], device=DEV), torch.tensor([[1.0, 0], [0, 1.0]], device=DEV), 2, 1.0)
    layer.set_slot_lora(1, torch.tensor([[0, 0, 1.0]], device=DEV), torch.tensor([[2.0], [4.0]], device=DEV), 1, 0.25)
    x = torch.tensor([[2.0, 3.0, 5.0], [7.0, 11.0, 13.0], [17.0, 19.0, 23.0]], device=DEV)
    assert not layer(x).any()
    CTX.set_lora_context(CTX.LoRAContext(
        token_to_slot=torch.tensor([0, -1, 1], dtype=torch.int32, device=DEV),
        token_indices_sorted_by_slot=torch.tensor([0, 2, 1], dtype=torch.int32, device=DEV),
        active_slot_ids=torch.tensor([0, 1], dtype=torch.int32, device=DEV),
        num_tokens_per_slot=torch.tensor([1, 1], dtype=torch.int32, device=DEV),
        slot_start_offsets=torch.tensor([0, 1, 2], dtype=torch.int32, device=DEV), no_lora_flag=False))
    assert layer(x).cpu().tolist() == [[2.0, 3.0], [0.0, 0.0], [11.5, 23.0]]

    merged = L.LoRAMergedColumnParallelLinear(2, [1, 1], lora_targets=[0], max_loras=1, max_lora_rank=1).to(DEV).half()
    merged.weight.data.zero_()
    merged.set_slot_lora(0, torch.tensor([[[1.0, 0.0]]], device=DEV, dtype=torch.float16),
                         [torch.tensor([[2.0]], device=DEV, dtype=torch.float16)], 1, 0.5)
    CTX.set_lora_context(CTX.build_lora_context_from_token_to_slot(torch.tensor([0], dtype=torch.int32, device=DEV)))
    assert merged(torch.tensor([[4.0, 8.0]], device=DEV, dtype=torch.float16)).cpu().tolist() == [[4.0, 0.0]]


def test_context_length_mismatch_raises_before_launch():
    layer = L.LoRALinear(32, 32, bias=False, max_loras=1, max_lora_rank=32).to(DEV).bfloat16()
    layer.set_slot_lora(0, torch.ones(32, 32, device=DEV), torch.ones(32, 32, device=DEV), 32, 1.0)
    CTX.set_lora_context(CTX.build_lora_context_from_token_to_slot(torch.zeros(3, dtype=torch.int32, device=DEV)))
    with pytest.raises(RuntimeError, match="length does not match"):
        layer(torch.ones(2, 32, device=DEV, dtype=torch.bfloat16))


# ------------------------------------------------------------------- CUDA graphs
def test_cuda_graph_replay_with_changing_slots_and_weights():
    """Graph contract of the runner (engine/model_runner.py:819-923): fixed grid over
    max_loras+1 buckets, metadata and slab contents change between capture and replay
    (tests/unit/test_lora_cuda.py:224-382,454-532)."""
    S, T = 8, 32
    layer = L.LoRAQKVParallelLinear(1024, 64, 16, 2, max_loras=S, max_lora_rank=32).to(DEV).bfloat16()
    g = torch.Generator().manual_seed(1)
    layer.weight.data.copy_(torch.randn(1280, 1024, generator=g) * 0.02)

    def load(slot, seed, rank):
        gg = torch.Generator().manual_seed(seed)
        a = (torch.randn(3, rank, 1024, generator=gg) * 0.05).to(DEV)
        b = [(torch.randn(w, rank, generator=gg) * 0.05).to(DEV) for w in (1024, 128, 128)]
        layer.set_slot_lora(slot, a, b, rank, 1.0)

    for s in range(S):
        load(s, 100 + s, 32)
    bufs = BP.GraphLoRABuffers.make(T, S, device=DEV)
    x = torch.zeros(T, 1024, device=DEV, dtype=torch.bfloat16)
    out = torch.zeros(T, 1280, device=DEV, dtype=torch.bfloat16)
    bufs.load_plan(BP.build_lora_batch_plan_from_token_to_slot({}, [0] * T))  # capture with every row on slot 0
    CTX.set_lora_context(bufs.context(T))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.no_grad():
        layer(x)  # warm-up outside capture
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.no_grad(), torch.cuda.graph(graph):
        out.copy_(layer(x))

    def eager_reference(slots, xin):
        CTX.set_lora_context(BP.build_lora_context_from_slot_list(slots, device=DEV))
        with torch.no_grad():
            return layer(xin).clone()

    for step, slots in enumerate([[(i * 3) % S if i % 5 else -1 for i in range(T)], [-1] * T, [S - 1] * T]):
        if step == 2:
            load(S - 1, 999, 16)  # slot rewritten between capture and replay
        x.copy_((torch.randn(T, 1024, generator=g)).to(torch.bfloat16))
        bufs.load_plan(BP.build_lora_batch_plan_from_token_to_slot({}, slots))
        graph.replay()
        torch.cuda.synchronize()
        want = eager_reference(slots, x)
        assert torch.equal(out, want), f"graph replay differs from eager at step {step}"
        a_slabs = [layer.lora_A.data[i].cpu() for i in range(3)]
        b_slabs = [getattr(layer, f"lora_B_{t}").data.cpu() for t in "qkv"]
        base = (x.float().cpu() @ layer.weight.data.float().cpu().T).to(torch.bfloat16)
        ref = O.add_lora(base, x.cpu(), a_slabs, b_slabs, slots, 1.0, [0, 1024, 1152])
        assert_lora_close(out, ref, max_abs=4e-2, what=f"graph step {step}")  # base GEMM rounding included


# ------------------------------------------------------------------ prefill SGMV (tcgen05)
@pytest.mark.parametrize("name", ["qkv", "o", "gate_up", "down"])
def test_prefill_projection_matches_oracle(name):
    """Prefill config at reduced length (5 requests, 602 rows, mixed ranks 8/16/64 in a rank-64 slab):
    tensor-core kernels vs oracle; rows of a request boundary share a 128-row block."""
    p = W.prefill_projection(name, seed=3, lengths=[200, 77, 133, 128, 64])
    p.token_to_slot[10:25] = -1  # a hole without adapter inside the first request
    # bit patterns that an "add zero" would destroy: -0.0, a bf16 denormal, the largest finite value
    p.y[10:25, 0::3] = -0.0
    p.y[10:25, 1::3] = torch.tensor(1e-40).to(torch.bfloat16)
    p.y[12, 5] = torch.finfo(torch.bfloat16).max
    out, y_in = run_add(p, N.IMPL_SGMV)
    check_against_oracle(p, out, y_in, what=f"sgmv/{name}")
    out2, _ = run_add(p, N.IMPL_SGMV)
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16)), "two runs differ bitwise"
    auto, _ = run_add(p, N.IMPL_AUTO)  # 602 rows >= 512: auto picks the prefill kernels
    assert torch.equal(out.view(torch.int16), auto.view(torch.int16))


@pytest.mark.parametrize("r_max", [16, 32, 64])
def test_sgmv_ranks_scales_strides_and_ragged_length(r_max):
    lengths = [130, 1, 255, 7, 64]  # T = 457: not a multiple of 128, runs of length 1 and 7
    slots = []
    for i, n in enumerate(lengths):
        slots += [i % 3] * n
    p = W.make_projection(17 + r_max, len(slots), 512, [384, 0, 128], 3, r_max, token_to_slot=slots)
    p.a_slabs[1] = p.a_slabs[0]
    sps = torch.tensor([1.0, 0.5, 2.0])
    out, y_in = run_add(p, N.IMPL_SGMV, scaling=0.5, scale_per_slot=sps, y_pad=16, x_pad=8)
    check_against_oracle(p, out, y_in, 0.5, sps, what=f"sgmv r={r_max}")


def test_sgmv_random_slots_and_full_size_properties():
    # decode-like random map through the prefill kernels: many one-row runs per block (slow path, still exact)
    p = W.make_projection(23, 200, 256, [256], 8, 32, p_none=0.2)
    out, y_in = run_add(p, N.IMPL_SGMV)
    check_against_oracle(p, out, y_in, what="sgmv random slots")


@pytest.mark.parametrize("name", ["qkv", "o", "gate_up", "down"])
def test_prefill_config_full_size_matches_oracle(name):
    """The prefill configuration at its full size (16 requests packed to 8172 rows, hidden 2048, intermediate
    6144, ranks 8 / 16 / 64 in rank-64 slabs): the tensor-core add, the overwrite form and the fused base GEMM
    against the fp32 oracle, rows without adapter bit-exact in all three."""
    p = W.prefill_projection(name, seed=0)
    assert p.x.shape[0] > 8000
    p.token_to_slot[300:391] = -1  # a hole without adapter across a 128-row block boundary
    p.token_to_slot[-17:] = -1     # and a ragged tail
    none = p.token_to_slot < 0
    # --- y += delta
    out, y_in = run_add(p, N.IMPL_SGMV)
    check_against_oracle(p, out, y_in, what=f"sgmv add / {name} / full size")
    # --- y = delta (-0.0 in rows without adapter)
    d = p.to_device(DEV)
    S = d.a_slabs[0].shape[0]
    delta = torch.full_like(d.y, 7.0)
    LORA.launch_add(delta, d.x, d.a_slabs, d.b_slabs, d.out_sizes, d.col_offsets, metadata_for(d.token_to_slot, "eager", S),
                    1.0, impl=N.IMPL_SGMV, overwrite=True)
    torch.cuda.synchronize()
    want = O.add_lora(torch.zeros_like(p.y), p.x, p.a_slabs, p.b_slabs, p.token_to_slot, 1.0, p.col_offsets)
    assert_lora_close(delta.cpu(), want, what=f"sgmv delta / {name} / full size")
    assert bool((delta.cpu()[none].view(torch.int16) == -32768).all()), "rows without adapter are not -0.0"
    # --- y = x @ W.T + delta in one kernel; the base weight is scaled so that outputs stay of order one
    #     (|y| < 4) and the path's own absolute bound is the one tested, rounding of the base included
    gen = torch.Generator().manual_seed(99)
    weight = (torch.randn(sum(p.out_sizes), p.x.shape[1], generator=gen) * (0.5 / p.x.shape[1] ** 0.5)).to(torch.bfloat16)
    base = p.x.float() @ weight.float().T
    ref = O.add_lora(base, p.x, p.a_slabs, p.b_slabs, p.token_to_slot, 1.0, p.col_offsets)
    w_dev = weight.to(DEV)
    fused = LORA.linear_lora(d.x, w_dev, None, d.a_slabs, d.b_slabs, d.out_sizes, d.col_offsets, d.token_to_slot, 1.0)
    plain = LORA.linear_lora(d.x, w_dev, None, d.a_slabs, d.b_slabs, d.out_sizes, d.col_offsets, None, 1.0)
    torch.cuda.synchronize()
    assert N.device_status(reset=True) == 0
    assert float(ref.abs().max()) < 4.0
    assert_lora_close(fused.cpu(), ref, what=f"fused linear / {name} / full size")
    assert_lora_close(plain.cpu(), base, what=f"plain linear / {name} / full size")
    none_d = none.to(DEV)
    assert torch.equal(fused[none_d].view(torch.int16), plain[none_d].view(torch.int16)), "rows with slot -1 changed"
    assert not torch.equal(fused[~none_d], plain[~none_d])


def test_sgmv_unsupported_and_workspace_errors():
    p = W.make_projection(4, 64, 96, [64], 2, 32)  # in % 64 != 0
    with pytest.raises(RuntimeError, match="prefill kernels"):
        run_add(p, N.IMPL_SGMV)
    d = W.make_projection(4, 64, 128, [64], 2, 32).to_device(DEV)
    meta = metadata_for(d.token_to_slot, "eager", 2)
    tiny = torch.empty(16, dtype=torch.uint8, device=DEV)
    with pytest.raises(RuntimeError, match="scratch"):
        LORA.launch_add(d.y, d.x, d.a_slabs, d.b_slabs, d.out_sizes, d.col_offsets, meta, 1.0, impl=N.IMPL_SGMV, workspace=tiny)
    assert N.workspace_bytes(8192, 3, 64) >= 3 * 8192 * 64 * 2


# ------------------------------------------------------------------ fused base GEMM + LoRA (tcgen05)
def run_linear(p: W.Projection, bias=None, slots="own", **kw):
    d = p.to_device(DEV)
    tts = d.token_to_slot if slots == "own" else slots
    out = LORA.linear_lora(d.x, d.weight, None if bias is None else bias.to(DEV), d.a_slabs, d.b_slabs,
                           d.out_sizes, d.col_offsets, tts, 1.0, **kw)
    torch.cuda.synchronize()
    assert N.device_status(reset=True) == 0
    return out


@pytest.mark.parametrize("r_max,outs,bias", [(64, [512], False), (32, [256, 128, 128], True), (16, [384, 0, 128], True)])
def test_fused_linear_lora_matches_oracle(r_max, outs, bias):
    """One kernel computes x @ W.T (+ bias) and the LoRA delta; rows without adapter are
    bit-identical to the same kernel run without any LoRA."""
    lengths = [300, 128, 77, 1, 250, 140]  # T = 896: blocks with one slot, several slots and -1 holes
    slots = []
    for i, n in enumerate(lengths):
        slots += [(i * 2) % 5] * n
    p = W.make_projection(31 + r_max, len(slots), 1024, outs, 5, r_max, token_to_slot=slots, with_weight=True,
                          ranks=[r_max, r_max // 2, r_max, 8, r_max])
    p.token_to_slot[40:90] = -1
    p.token_to_slot[600:603] = -1
    gen = torch.Generator().manual_seed(5)
    b = (torch.randn(sum(outs), generator=gen) * 0.5).to(torch.bfloat16) if bias else None
    active = [i for i, w in enumerate(outs) if w > 0]
    q = W.Projection(p.x, p.y, [p.a_slabs[i] for i in active], [p.b_slabs[i] for i in active],
                     [outs[i] for i in active], [p.col_offsets[i] for i in active], p.ranks, p.token_to_slot, p.weight)
    out = run_linear(q, b)
    ref = O.linear_lora(q.x, q.weight, b, q.a_slabs, q.b_slabs, q.col_offsets, q.token_to_slot)
    assert_lora_close(out, ref, max_abs=4e-2, what=f"fused linear r={r_max}")  # bf16 rounding of the base output included
    plain = run_linear(q, b, slots=None)
    assert_lora_close(plain, O.linear_lora(q.x, q.weight, b, None, None, None, None), max_abs=4e-2, what="plain linear")
    none = (q.token_to_slot < 0).to(DEV)
    assert torch.equal(out[none].view(torch.int16), plain[none].view(torch.int16)), "rows with slot -1 changed"
    assert not torch.equal(out[~none], plain[~none])
    again = run_linear(q, b)
    assert torch.equal(out.view(torch.int16), again.view(torch.int16)), "two runs differ bitwise"


def test_fused_linear_ragged_shapes_and_strides():
    # T not a multiple of 128, out not a multiple of 256, padded row strides, caller-provided output
    p = W.make_projection(9, 517, 320, [200, 120], 3, 32, with_weight=True, p_none=0.3)
    d = p.to_device(DEV)
    xp = torch.zeros(517, 320 + 64, dtype=torch.bfloat16, device=DEV)
    xp[:, :320] = d.x
    wp = torch.zeros(320, 320 + 8, dtype=torch.bfloat16, device=DEV)
    wp[:, :320] = d.weight
    out = torch.full((517, 320 + 16), 7.0, dtype=torch.bfloat16, device=DEV)
    got = LORA.linear_lora(xp[:, :320], wp[:, :320], None, d.a_slabs, d.b_slabs, d.out_sizes, d.col_offsets,
                           d.token_to_slot, 1.0, out=out[:, :320])
    torch.cuda.synchronize()
    assert got.data_ptr() == out.data_ptr()
    ref = O.linear_lora(p.x, p.weight, None, p.a_slabs, p.b_slabs, p.col_offsets, p.token_to_slot)
    assert_lora_close(out[:, :320], ref, max_abs=4e-2, what="fused linear, ragged")
    assert bool((out[:, 320:] == 7.0).all()), "columns beyond the output were written"


def test_layers_take_fused_linear_when_switched_on(monkeypatch):
    case = dict(kind="merged", hidden=512, outs=[768, 768], S=4, r=32)
    torch.manual_seed(3)
    layer = L.LoRAMergedColumnParallelLinear(case["hidden"], case["outs"], max_loras=4, max_lora_rank=32).to(DEV, torch.bfloat16)
    layer.weight.data.normal_(0, 0.02)
    for s in range(3):
        a = torch.randn(2, 32, 512) * 0.05
        bs = [torch.randn(768, 32) * 0.05, torch.randn(768, 32) * 0.05]
        layer.set_slot_lora(s, a, bs, 32, 1.5)
    T = 640
    slots = torch.tensor(([0] * 200 + [-1] * 56 + [2] * 256 + [1] * 128), dtype=torch.int32)
    x = torch.randn(T, 512).to(torch.bfloat16).to(DEV)
    CTX.set_lora_context(CTX.build_lora_context_from_token_to_slot(slots.to(DEV)))
    calls = []
    real = LORA.linear_lora
    monkeypatch.setattr(LORA, "linear_lora", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    with torch.no_grad():
        unfused = layer(x)
        assert not calls
        monkeypatch.setattr(L, "FUSED_LINEAR", True)
        fused = layer(x)
        assert calls == [1]
    torch.cuda.synchronize()
    assert_lora_close(fused, unfused.float(), max_abs=4e-2, what="fused vs cuBLAS + add")
    assert not torch.equal(fused[:200], (x[:200] @ layer.weight.T))


# ------------------------------------------------------------------ device-side metadata build
def _random_map(seed, T, S, p_none):
    gen = torch.Generator().manual_seed(seed)
    return W.uniform_slots(gen, T, S, p_none)


@pytest.mark.parametrize("T,S,p_none", [(1, 4, 0.0), (256, 32, 0.1), (777, 5, 0.5), (1024, 128, 0.02), (4096, 16, 0.3),
                                        (8172, 16, 0.0), (16384, 1024, 0.1), (300, 4095, 0.2), (64, 8, 1.0)])
def test_device_metadata_build_is_bit_identical_to_the_host_builders(T, S, p_none):
    slots = _random_map(T + S, T, S, p_none)
    if T == 8172:  # prefill layout: contiguous requests, one slot each
        slots = W.prefill_projection("o", seed=0).token_to_slot
    dev = slots.to(DEV)
    # --- graph buffers (stale tail of the sorted buffer must stay as it was)
    rows = min(T + 7, 16384)  # buffers longer than the step, as the runner's are
    host = BP.GraphLoRABuffers.make(rows, S, device=DEV)
    host.load_plan(BP.build_lora_batch_plan_from_token_to_slot({}, slots.tolist()))
    mine = BP.GraphLoRABuffers.make(rows, S, device=DEV)
    mine.load_token_to_slot_on_device(dev)
    torch.cuda.synchronize()
    for name in ("token_to_slot", "token_indices_sorted_by_slot", "active_slot_ids", "num_tokens_per_slot", "slot_start_offsets"):
        assert torch.equal(getattr(mine, name), getattr(host, name)), f"graph buffers: {name} differs"
    # --- vLLM-style kernel metadata
    km_host = LoRAKernelMeta.make(S, T, DEV)
    km_host.prepare_tensors(dev)
    km_dev = LoRAKernelMeta.make(S, T, DEV)
    km_dev.token_indices_sorted_by_lora_ids.copy_(km_host.token_indices_sorted_by_lora_ids)  # same uninitialised tail
    km_dev.token_lora_mapping.copy_(km_host.token_lora_mapping)
    km_dev.active_lora_ids.fill_(7)
    km_dev.num_tokens_per_lora.fill_(7)
    km_dev.lora_token_start_loc.fill_(7)
    km_dev.prepare_tensors_on_device(dev)
    torch.cuda.synchronize()
    for name in ("token_indices_sorted_by_lora_ids", "active_lora_ids", "num_tokens_per_lora", "lora_token_start_loc"):
        a, b = getattr(km_dev, name), getattr(km_host, name)
        if name == "token_indices_sorted_by_lora_ids" and p_none == 1.0:
            continue  # the host builder returns before it writes the order
        assert torch.equal(a, b), f"kernel meta: {name} differs"
    # --- eager plan (compact, no -1 bucket)
    plan = BP.build_lora_batch_plan_from_token_to_slot({}, slots.tolist())
    srt = torch.full((T,), -5, dtype=torch.int32, device=DEV)
    ids = torch.empty(S + 1, dtype=torch.int32, device=DEV)
    cnt = torch.empty(S + 1, dtype=torch.int32, device=DEV)
    off = torch.empty(S + 2, dtype=torch.int32, device=DEV)
    info = torch.zeros(3, dtype=torch.int32, device=DEV)
    N.build_metadata(dev, S, N.META_EAGER, srt, ids, cnt, off, info)
    k, rows, bad = info.tolist()
    assert (k, rows, bad) == (len(plan.active_slot_ids), len(plan.token_indices_sorted_by_slot), 0)
    assert srt[:rows].tolist() == list(plan.token_indices_sorted_by_slot) and bool((srt[rows:] == -5).all())
    assert ids[:k].tolist() == list(plan.active_slot_ids) and bool((ids[k:] == -1).all())
    assert cnt[:k].tolist() == list(plan.num_tokens_per_slot) and bool((cnt[k:] == 0).all())
    assert off[: k + 1].tolist() == list(plan.slot_start_offsets) and bool((off[k + 1:] == 0).all())


def test_device_metadata_feeds_the_decode_kernel_and_reports_bad_ids():
    p = W.decode_projection("qkv", seed=21)
    d = p.to_device(DEV)
    bufs = BP.GraphLoRABuffers.make(256, 32, device=DEV)
    bufs.load_token_to_slot_on_device(d.token_to_slot)
    ctx = bufs.context(256)
    meta = LORA.LoRAMetadata(ctx.token_to_slot, ctx.token_indices_sorted_by_slot, ctx.active_slot_ids,
                             ctx.num_tokens_per_slot, ctx.slot_start_offsets, False, ctx.num_active_loras)
    y = d.y.clone()
    LORA.launch_add(y, d.x, d.a_slabs, d.b_slabs, d.out_sizes, d.col_offsets, meta, 1.0, impl=N.IMPL_BGMV)
    torch.cuda.synchronize()
    check_against_oracle(p, y.cpu(), p.y, what="decode kernel on device-built graph buffers")
    # ids outside [-1, S) are counted and treated as "no adapter"
    bad = torch.tensor([0, 1, 9, -3, 1, -1], dtype=torch.int32, device=DEV)
    srt = torch.empty(6, dtype=torch.int32, device=DEV)
    cnt = torch.empty(3, dtype=torch.int32, device=DEV)
    off = torch.empty(4, dtype=torch.int32, device=DEV)
    info = torch.zeros(3, dtype=torch.int32, device=DEV)
    N.build_metadata(bad, 2, N.META_GRAPH, srt, None, cnt, off, info)
    assert info.tolist() == [3, 3, 2] and cnt.tolist() == [0, 1, 2] and off.tolist() == [0, 0, 1, 3] and srt[:3].tolist() == [0, 1, 4]
    with pytest.raises(RuntimeError, match="metadata build"):
        N.build_metadata(torch.zeros(20000, dtype=torch.int32, device=DEV), 2, N.META_GRAPH,
                         torch.empty(20000, dtype=torch.int32, device=DEV), None, cnt, off, None)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        N.build_metadata(torch.zeros(4, dtype=torch.int32), 2, N.META_GRAPH, srt, None, cnt, off, None)
