"""Adapter admission through one packed copy + one kernel against the layers' own module-by-module
``set_slot_lora`` path: slabs and per-slot buffers must be bit-identical."""

import copy

import pytest
import torch

from nanovllm_voxcpm_b200 import _native as N
from nanovllm_voxcpm_b200 import backbone as BB
from nanovllm_voxcpm_b200 import layers as L
from nanovllm_voxcpm_b200.slot_loader import SlotLoader
from oracle import lora_oracle as O

pytestmark = pytest.mark.gpu


def _model():
    cfg = BB.DecoderConfig(hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=512,
                           num_layers=2, max_loras=4, max_lora_rank=32, max_position=64)
    with torch.device("cuda"):
        model = BB.Decoder(cfg).to(torch.bfloat16)
    return cfg, model


def _adapter(model, rank, scaling, seed, payload_rank=None, dtype=torch.float32, skip=()):
    """Random payload in the form each layer's set_slot_lora takes (host tensors)."""
    gen = torch.Generator().manual_seed(seed)
    pr = payload_rank or rank
    out = {}
    for name, m in model.named_modules():
        if not isinstance(m, L._LORA_LAYER_TYPES) or any(s in name for s in skip):
            continue
        a_slabs, b_slabs = m._a_slices(), m._b_slices()
        a = [torch.randn(pr, s.size(2), generator=gen).to(dtype) * 0.1 for s in a_slabs]
        b = [torch.randn(s.size(1), pr, generator=gen).to(dtype) * 0.1 for s in b_slabs]
        if len(a_slabs) > 1:
            out[name] = (torch.stack(a), b, rank, scaling)
        else:
            out[name] = (a[0], b[0], rank, scaling)
    return out


def _state(model):
    st = {}
    for name, m in model.named_modules():
        if isinstance(m, L._LORA_LAYER_TYPES):
            for i, t in enumerate((*m._a_slices(), *m._b_slices())):
                st[f"{name}.slab{i}"] = t.detach().clone()
            st[f"{name}.rank"] = m.effective_lora_rank.clone()
            st[f"{name}.scaling"] = m.lora_scaling.clone()
            st[f"{name}.base_scaling"] = m.lora_base_scaling.clone()
            st[f"{name}.host"] = (list(m._effective_lora_rank_values), list(m._lora_scaling_values))
    return st


def _load_by_module(model, slot, payload):
    for name, m in model.named_modules():
        if name in payload:
            a, b, rank, sc = payload[name]
            m.set_slot_lora(slot, a.cuda(), [t.cuda() for t in b] if isinstance(b, list) else b.cuda(), rank, sc)


def test_batched_slot_load_equals_module_by_module_load():
    cfg, model = _model()
    ref = copy.deepcopy(model)
    loader = SlotLoader(model)
    steps = [
        (1, _adapter(model, 32, 1.5, seed=1)),
        (3, _adapter(model, 8, 0.25, seed=2, payload_rank=16)),                       # payload wider than the rank used
        (1, _adapter(model, 16, 2.0, seed=3, dtype=torch.bfloat16, skip=("mlp",))),   # replaces slot 1, covers attention only
        (0, _adapter(model, 4, 0.5, seed=4, dtype=torch.float16)),
    ]
    cleared_by_runner = {}
    # third witness: the oracle's slab writer on host copies of the (all-zero) slabs
    lora_mods = {n: m for n, m in model.named_modules() if isinstance(m, L._LORA_LAYER_TYPES)}
    oracle_slabs = {n: ([torch.zeros_like(t, device="cpu") for t in m._a_slices()],
                        [torch.zeros_like(t, device="cpu") for t in m._b_slices()]) for n, m in lora_mods.items()}
    for slot, payload in steps:
        for name in cleared_by_runner.get(slot, []):
            for t in (*oracle_slabs[name][0], *oracle_slabs[name][1]):
                t[slot].zero_()
        for name, (a, b, rank, sc) in payload.items():
            a_list = list(a) if isinstance(b, list) else [a]
            b_list = b if isinstance(b, list) else [b]
            for a_slab, b_slab, a_i, b_i in zip(*oracle_slabs[name], a_list, b_list):
                O.write_slot(a_slab, b_slab, slot, a_i, b_i, rank, sc)
        loader.load_slot(slot, payload)
        # the reference path: clear what the previous occupant loaded, then module by module
        for name in cleared_by_runner.get(slot, []):
            dict(ref.named_modules())[name].clear_slot_lora(slot)
        _load_by_module(ref, slot, payload)
        cleared_by_runner[slot] = list(payload)
        torch.cuda.synchronize()
        got, want = _state(model), _state(ref)
        for key in want:
            if key.endswith(".host"):
                assert got[key] == want[key], key
            else:
                assert torch.equal(got[key], want[key]), f"{key} differs after loading slot {slot}"
        for name, m in lora_mods.items():
            for i, (t, want_t) in enumerate(zip((*m._a_slices(), *m._b_slices()), (*oracle_slabs[name][0], *oracle_slabs[name][1]))):
                assert torch.equal(t.cpu(), want_t), f"{name} slab {i} differs from the oracle's writer after loading slot {slot}"
    assert N.device_status() == 0
    with pytest.raises(ValueError, match="Unknown LoRA target module"):
        loader.load_slot(0, {"nope": steps[0][1][next(iter(steps[0][1]))]})
    with pytest.raises(ValueError):
        bad = _adapter(model, 64, 1.0, seed=5)  # rank above max_lora_rank
        loader.load_slot(0, bad)


def test_checkpoint_payload_is_admitted_from_its_arena(tmp_path):
    """Checkpoint on disk -> one pinned arena -> slot: same slabs as loading the same payload module by module."""
    from nanovllm_voxcpm_b200 import adapter_checkpoint as ac

    cfg, model = _model()
    ref = copy.deepcopy(model)
    gen = torch.Generator().manual_seed(11)
    rank, tensors = 16, {}
    unpack = {"qkv_proj": ("q_proj", "k_proj", "v_proj"), "gate_up_proj": ("gate_proj", "up_proj")}
    for name, m in model.named_modules():
        if not isinstance(m, L._LORA_LAYER_TYPES):
            continue
        parent, _, leaf = name.rpartition(".")
        for proj, a_slab, b_slab in zip(unpack.get(leaf, (leaf,)), m._a_slices(), m._b_slices()):
            tensors[f"base_model.model.{parent}.{proj}.lora_A"] = (torch.randn(rank, a_slab.size(2), generator=gen) * 0.1).bfloat16()
            tensors[f"base_model.model.{parent}.{proj}.lora_B"] = (torch.randn(b_slab.size(1), rank, generator=gen) * 0.1).bfloat16()
    path = ac.save_lora_checkpoint(str(tmp_path / "adapter"), tensors, rank=rank, alpha=24.0)
    payload = ac.load_lora_checkpoint(str(path))
    assert payload.arena.is_pinned() and payload.modules.keys() == {n for n, m in model.named_modules()
                                                                    if isinstance(m, L._LORA_LAYER_TYPES)}
    loader = SlotLoader(model)
    loader.load_slot(2, _adapter(model, 32, 1.0, seed=12))  # an occupant to replace
    loader.load_slot(2, payload)
    loader.load_slot(0, payload)  # the same payload again: its cached descriptor table, aimed at another slot
    assert len(loader._plans) == 1
    by_name = {n: (m.lora_a, m.lora_b, m.effective_rank, m.scaling) for n, m in payload.modules.items()}
    _load_by_module(ref, 2, by_name)
    _load_by_module(ref, 0, by_name)
    torch.cuda.synchronize()
    got, want = _state(model), _state(ref)
    for key in want:
        if key.endswith(".host"):
            assert got[key] == want[key], key
        else:
            assert torch.equal(got[key], want[key]), key
    assert N.device_status() == 0
