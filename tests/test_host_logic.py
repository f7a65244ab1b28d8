"""Host-side logic on the CPU: metadata builders against the reference-generated
fixtures, the layer classes (slot loading, gating, TP sharding, errors) with the oracle
standing in for the kernels, and the backend's pre-launch error contract."""

import numpy as np
import pytest
import torch

import cases
from helpers import OracleBackend, build_b200_layer, load_golden
from nanovllm_voxcpm_b200 import batch_plan as BP
from nanovllm_voxcpm_b200 import context as CTX
from nanovllm_voxcpm_b200 import layers as L
from nanovllm_voxcpm_b200 import lora as LORA
from nanovllm_voxcpm_b200.lora_ops import LoRAKernelMeta


@pytest.fixture(autouse=True)
def _oracle_backend():
    LORA.set_backend_for_testing(OracleBackend())
    yield
    LORA.set_backend_for_testing(None)
    CTX.reset_lora_context()


@pytest.mark.parametrize("idx", range(len(cases.METADATA_CASES)))
def test_metadata_builders_match_reference(idx):
    g = load_golden("metadata.npz")
    max_loras, slots = cases.METADATA_CASES[idx]
    plan = BP.build_lora_batch_plan_from_token_to_slot({}, list(slots))
    assert plan.token_indices_sorted_by_slot == g[f"{idx}/plan_sorted"].tolist()
    assert plan.active_slot_ids == g[f"{idx}/plan_active"].tolist()
    assert plan.num_tokens_per_slot == g[f"{idx}/plan_counts"].tolist()
    assert plan.slot_start_offsets == g[f"{idx}/plan_offsets"].tolist()

    ctx = CTX.build_lora_context_from_token_to_slot(torch.tensor(slots, dtype=torch.int32))
    assert [int(ctx.no_lora_flag), ctx.num_active_loras] == g[f"{idx}/ctx_no_lora"].tolist()
    if not ctx.no_lora_flag:
        for key in ("token_indices_sorted_by_slot", "active_slot_ids", "num_tokens_per_slot", "slot_start_offsets"):
            got = getattr(ctx, key)
            assert got.dtype == torch.int32
            assert got.tolist() == g[f"{idx}/ctx_{key}"].tolist(), key

    dev = BP.build_lora_context_from_batch_plan(plan, device="cpu")
    assert dev.no_lora_flag == (not plan.active_slot_ids)
    if plan.active_slot_ids:
        assert dev.token_indices_sorted_by_slot.tolist() == plan.token_indices_sorted_by_slot
        assert dev.slot_start_offsets.tolist() == plan.slot_start_offsets and dev.token_to_slot.dtype == torch.int32

    if slots:
        km = LoRAKernelMeta.make(max_loras=max_loras, max_num_tokens=len(slots), device="cpu")
        km.prepare_tensors(torch.tensor(slots, dtype=torch.int32))
        assert [int(km.no_lora_flag), km.num_active_loras] == g[f"{idx}/vllm_flags"].tolist()
        assert np.array_equal(km.active_lora_ids.numpy(), g[f"{idx}/vllm_ids"])
        assert np.array_equal(km.num_tokens_per_lora.numpy(), g[f"{idx}/vllm_counts"])
        assert np.array_equal(km.lora_token_start_loc.numpy(), g[f"{idx}/vllm_starts"])
        if not km.no_lora_flag:
            assert np.array_equal(km.token_indices_sorted_by_lora_ids.numpy(), g[f"{idx}/vllm_sorted"])
            args = km.meta_args(len(slots), specialize_active_lora=False)
            assert args[6] == max_loras + 1 and args[0].numel() == len(slots)

    if plan.active_slot_ids:
        bufs = BP.GraphLoRABuffers.make(len(slots) + 3, max_loras, device="cpu")
        assert bufs.active_slot_ids.tolist() == list(range(-1, max_loras))
        bufs.load_plan(plan)
        assert np.array_equal(bufs.token_to_slot.numpy(), g[f"{idx}/graph_token_to_slot"])
        assert np.array_equal(bufs.token_indices_sorted_by_slot.numpy(), g[f"{idx}/graph_token_indices_sorted_by_slot"])
        assert np.array_equal(bufs.num_tokens_per_slot.numpy(), g[f"{idx}/graph_num_tokens_per_slot"])
        assert np.array_equal(bufs.slot_start_offsets.numpy(), g[f"{idx}/graph_slot_start_offsets"])
        gctx = bufs.context(len(slots))
        assert gctx.num_active_loras == max_loras + 1 and gctx.token_to_slot.numel() == len(slots)


def test_expand_token_counts():
    assert BP.expand_token_counts([0, -1, 0], [2, 1, 1]) == [0, 0, -1, 0]


@pytest.mark.parametrize("case", cases.LAYER_CASES, ids=lambda c: c["name"])
def test_layers_match_reference_with_oracle_backend(case):
    g = load_golden("layers.npz")
    inputs = cases.build_inputs(case)
    saved = L.dist.all_reduce
    L.dist.all_reduce = lambda t, *a, **k: t  # keep the per-rank partial of row-parallel layers
    try:
        for rank in range(case.get("tp", 1)):
            layer, x = build_b200_layer(L, case, inputs, rank)
            CTX.set_lora_context(CTX.build_lora_context_from_token_to_slot(inputs["slots"]))
            with torch.no_grad():
                y = layer(x)
            torch.testing.assert_close(y, torch.from_numpy(g[f"{case['name']}/y_rank{rank}"]), atol=2e-5, rtol=1e-5)
            # without a context the layer is the base linear
            CTX.reset_lora_context()
            with torch.no_grad():
                base = layer(x)
            none = inputs["slots"] < 0
            assert torch.equal(y[none], base[none])
    finally:
        L.dist.all_reduce = saved
    L._get_world_size = lambda: 1
    L._get_rank = lambda: 0


def test_slot_bookkeeping_and_padding():
    layer = L.LoRALinear(4, 3, bias=False, max_loras=2, max_lora_rank=4)
    layer.set_slot_lora(1, torch.ones(2, 4), torch.ones(3, 2), effective_rank=2, scaling=0.5)
    assert layer.effective_lora_rank.tolist() == [0, 2] and layer._effective_lora_rank_values == [0, 2]
    assert layer.lora_scaling.tolist() == [0.0, 0.5]
    assert torch.equal(layer.lora_A.data[1, 2:], torch.zeros(2, 4))  # zero padding beyond the rank
    assert torch.equal(layer.lora_B.data[1, :, :2], torch.full((3, 2), 0.5))  # scaling folded into B
    assert torch.equal(layer.lora_B.data[1, :, 2:], torch.zeros(3, 2))
    layer.clear_slot_lora(1)
    assert not layer.lora_A.data.any() and not layer.lora_B.data.any() and layer._effective_lora_rank_values == [0, 0]
    assert [m for m in L.iter_lora_modules(torch.nn.Sequential(layer, L.LoRALinear(2, 2)))] == [layer]
    assert set(L.get_lora_state_dict(layer)) == {"lora_A", "lora_B"}


def test_payload_validation_errors():
    lin = L.LoRALinear(4, 3, bias=False, max_loras=1, max_lora_rank=2)
    with pytest.raises(ValueError):  # rank above the slab (tests/unit/test_lora_layers.py:311-322)
        lin.set_slot_lora(0, torch.ones(3, 4), torch.ones(3, 3), effective_rank=3, scaling=1.0)
    with pytest.raises(ValueError):
        lin.validate_slot_lora_payload(torch.ones(2, 5), torch.ones(3, 2), 2, 1.0)
    with pytest.raises(ValueError):
        lin.validate_slot_lora_payload(torch.ones(2, 4), [torch.ones(3, 2)], 2, 1.0)
    with pytest.raises(ValueError):
        lin.validate_slot_lora_payload(torch.ones(2, 4), torch.ones(3, 2), 2, float("inf"))
    with pytest.raises(ValueError):
        L.LoRALinear(4, 3).validate_slot_lora_payload(torch.ones(2, 4), torch.ones(3, 2), 2, 1.0)
    qkv = L.LoRAQKVParallelLinear(8, 2, 2, 1, max_loras=1, max_lora_rank=2)
    qkv.validate_slot_lora_payload(torch.ones(3, 2, 8), [torch.ones(4, 2), torch.ones(2, 2), torch.ones(2, 2)], 2, 1.0)
    with pytest.raises(ValueError):
        qkv.validate_slot_lora_payload(torch.ones(3, 2, 8), torch.ones(4, 2), 2, 1.0)
    with pytest.raises(ValueError):
        qkv.validate_slot_lora_payload(torch.ones(3, 2, 8), [torch.ones(4, 2), torch.ones(3, 2), torch.ones(2, 2)], 2, 1.0)


def test_context_length_mismatch_raises_before_launch():
    """tests/unit/test_lora_cuda.py:192-221: RuntimeError before any kernel is launched."""
    layer = L.LoRALinear(4, 3, bias=False, max_loras=1, max_lora_rank=2)
    layer.weight.data.zero_()
    layer.set_slot_lora(0, torch.ones(2, 4), torch.ones(3, 2), 2, 1.0)
    CTX.set_lora_context(CTX.build_lora_context_from_token_to_slot(torch.tensor([0, 0, 0], dtype=torch.int32)))
    with pytest.raises(RuntimeError, match="length does not match"):
        layer(torch.ones(2, 4))


def test_empty_module_shortcut_and_domains():
    layer = L.LoRALinear(2, 1, bias=False, max_loras=2, max_lora_rank=1, lora_domain=CTX.PROJ_LORA_DOMAIN)
    layer.weight.data.zero_()
    CTX.set_lora_context(CTX.build_lora_context_from_token_to_slot(torch.tensor([0, 0, 0], dtype=torch.int32)))
    CTX.set_lora_context(
        CTX.build_lora_context_from_token_to_slot(torch.tensor([1], dtype=torch.int32)), domain=CTX.PROJ_LORA_DOMAIN
    )
    x = torch.tensor([[3.0, 5.0]])
    assert layer(x).item() == 0.0  # no slot resident in this module: op skipped
    layer.set_slot_lora(1, torch.tensor([[1.0, 0.0]]), torch.tensor([[2.0]]), 1, 1.0)
    assert layer(x).item() == 6.0  # tests/unit/test_lora_layers.py:186-233


def test_backend_error_contract_without_gpu():
    be = LORA.B200LoRABackend()
    assert be.availability().available is torch.cuda.is_available() or not be.availability().available
    y, x = torch.zeros(2, 4), torch.zeros(2, 4)
    a, b = torch.zeros(1, 2, 4), torch.zeros(1, 4, 2)
    meta = LORA.LoRAMetadata(torch.zeros(2, dtype=torch.int32), None, None, None, None, False, 0)
    assert be.add_lora([], x, [], [], indices=None, metadata=meta, scaling=1.0) == []
    with pytest.raises(ValueError, match="aligned"):
        be.add_lora([y], x, [a, a], [b], indices=None, metadata=meta, scaling=1.0)
    with pytest.raises(RuntimeError, match="metadata"):
        be.add_lora([y], x, [a], [b], indices=None, metadata=None, scaling=1.0)
    with pytest.raises(ValueError, match="contiguous"):
        be.add_lora([y], x, [a.transpose(1, 2)], [b], indices=None, metadata=meta, scaling=1.0)
    with pytest.raises(ValueError, match="2D"):
        be.add_lora([y], x, [a], [b], indices=None, metadata=meta, scaling=1.0, y_packed=torch.zeros(2, 2, 2))
    # no_lora_flag: silent no-op, same views back
    none = LORA.LoRAMetadata(torch.full((2,), -1, dtype=torch.int32), None, None, None, None, True, 0)
    assert be.add_lora([y], x, [a], [b], indices=None, metadata=none, scaling=1.0)[0] is y
    if not torch.cuda.is_available():
        # the product has no CPU path: CPU tensors are refused loudly
        with pytest.raises(RuntimeError, match="CUDA tensors only"):
            be.add_lora([y], x, [a], [b], indices=None, metadata=meta, scaling=1.0)
        LORA.set_backend_for_testing(None)
        assert LORA.is_available() is False
        with pytest.raises(RuntimeError):
            LORA.assert_available()


def test_metadata_slicing():
    meta = LORA.LoRAMetadata(torch.arange(6, dtype=torch.int32), torch.arange(6, dtype=torch.int32),
                             torch.tensor([0], dtype=torch.int32), torch.tensor([6], dtype=torch.int32),
                             torch.tensor([0, 6], dtype=torch.int32), False, 1)
    tts, srt, cnt, off, ids, flag, n = meta.as_kernel_metadata(4)
    assert tts.numel() == 4 and srt.numel() == 4 and cnt.tolist() == [6] and n == 1 and flag is False


def test_mixed_step_context_has_one_eager_plan_per_row_range():
    """A step of decode rows followed by prefill chunks: every range carries the metadata that the eager builder
    gives for its own rows, empty ranges are skipped, and the whole context is 'no adapter' only if every range is."""
    slots = torch.tensor([2, -1, 0, 2, 5, 5, 5, 5, -1, -1, 1, 1], dtype=torch.int32)
    ctx = CTX.build_mixed_lora_context(slots, [4, 4, 8])  # [0,4) decode, [4,4) empty, [4,8) chunk, [8,12) chunk
    assert [(lo, hi) for lo, hi, _ in ctx.parts] == [(0, 4), (4, 8), (8, 12)]
    assert not ctx.no_lora_flag and ctx.num_active_loras == 2
    assert torch.equal(ctx.token_to_slot, slots)
    for lo, hi, part in ctx.parts:
        want = CTX.build_lora_context_from_token_to_slot(slots[lo:hi])
        for name in ("token_to_slot", "token_indices_sorted_by_slot", "active_slot_ids", "num_tokens_per_slot",
                     "slot_start_offsets"):
            a, b = getattr(part, name), getattr(want, name)
            assert (a is None and b is None) or torch.equal(a, b), name
        assert part.no_lora_flag == want.no_lora_flag and part.num_active_loras == want.num_active_loras
        # row indices are relative to the range
        if part.token_indices_sorted_by_slot is not None:
            assert int(part.token_indices_sorted_by_slot.max()) < hi - lo
    none = CTX.build_mixed_lora_context(torch.full((6,), -1, dtype=torch.int32), [2])
    assert none.no_lora_flag and all(p[2].no_lora_flag for p in none.parts)


@pytest.mark.parametrize("case", [c for c in cases.LAYER_CASES if c.get("tp", 1) == 1], ids=lambda c: c["name"])
def test_layers_split_a_mixed_step_per_row_range(case):
    """With a mixed-step context the layers issue one multi-LoRA call per row range; the result equals the
    single-call result on the same rows (the op is row-wise)."""
    inputs = cases.build_inputs(case)
    layer, x = build_b200_layer(L, case, inputs, 0)
    T = x.shape[0]
    CTX.set_lora_context(CTX.build_lora_context_from_token_to_slot(inputs["slots"]))
    with torch.no_grad():
        whole = layer(x)
    CTX.set_lora_context(CTX.build_mixed_lora_context(inputs["slots"], [T // 3, T // 3, (2 * T) // 3]))
    with torch.no_grad():
        split = layer(x)
    CTX.reset_lora_context()
    torch.testing.assert_close(split, whole, atol=1e-6, rtol=1e-6)
