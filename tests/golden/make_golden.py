"""Generates tests/golden/*.npz by running the REFERENCE's own Python code on the CPU.

Run where the reference is importable:  PYTHONPATH=/path/to/reference python tests/golden/make_golden.py
(the reference cannot travel to the GPU box, the fixtures can).  What runs:
  * the reference layer classes (nanovllm_voxcpm/layers/lora.py) with the pure-PyTorch
    backend the reference's tests define (tests/unit/test_lora_layers.py:6-48), installed
    through nanovllm_voxcpm.lora.set_backend_for_testing;
  * the reference metadata builders (engine/lora_manager.py, utils/context.py,
    lora_ops/triton_ops/lora_kernel_metadata.py, engine/model_runner.py graph buffers).
Inputs come from tests/golden/cases.py and nanovllm_voxcpm_b200.workloads (seeded), so the
fixtures hold outputs plus input checksums only.
"""

from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("LORA_REFERENCE_ROOT") or (sys.argv[1] if len(sys.argv) > 1 else None)
if not REF or not os.path.isdir(REF):
    raise SystemExit("usage: LORA_REFERENCE_ROOT=<checkout of the reference project> python " + os.path.basename(__file__)
                     + "   (or pass the path as the first argument)")
sys.path.insert(0, ROOT)
sys.path.insert(0, REF)
sys.path.insert(0, HERE)

import cases  # noqa: E402
import nanovllm_voxcpm.layers.lora as ref_layers  # noqa: E402
import nanovllm_voxcpm.lora as ref_lora  # noqa: E402
from nanovllm_voxcpm.engine import lora_manager as ref_manager  # noqa: E402
from nanovllm_voxcpm.lora_ops.triton_ops.lora_kernel_metadata import LoRAKernelMeta  # noqa: E402
from nanovllm_voxcpm.utils import context as ref_context  # noqa: E402

from nanovllm_voxcpm_b200 import workloads  # noqa: E402


def _reference_test_backend():
    path = os.path.join(REF, "tests", "unit", "test_lora_layers.py")
    spec = importlib.util.spec_from_file_location("_ref_test_lora_layers", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod._FakePunicaBackend()


def checksum(*tensors) -> np.ndarray:
    return np.array([float(t.double().sum()) for t in tensors] + [float(t.double().abs().sum()) for t in tensors])


def run_reference_layer(case, inputs, tp_rank):
    tp = case.get("tp", 1)
    ref_layers._get_world_size = lambda: tp
    ref_layers._get_rank = lambda: tp_rank
    ref_layers.dist.all_reduce = lambda t, *a, **k: t  # keep the per-rank partial
    kind = case["kind"]
    S, r = case["S"], case["r_max"]
    if kind == "linear":
        layer = ref_layers.LoRALinear(case["in_f"], case["out_f"], bias=case["bias"], max_loras=S, max_lora_rank=r)
        layer.weight.data.copy_(inputs["weights"][0])
        if case["bias"]:
            layer.bias.data.copy_(inputs["bias"])
    elif kind == "row":
        layer = ref_layers.LoRARowParallelLinear(case["in_f"], case["out_f"], bias=case["bias"], max_loras=S, max_lora_rank=r)
        layer._base_weight_loader(layer.weight, inputs["weights"][0])
        if case["bias"]:
            layer._base_weight_loader(layer.bias, inputs["bias"])
    elif kind == "qkv":
        layer = ref_layers.LoRAQKVParallelLinear(
            case["hidden"], case["head"], case["heads"], case["kv_heads"], bias=False, lora_targets=case["targets"],
            max_loras=S, max_lora_rank=r,
        )
        for name, w in zip("qkv", inputs["weights"]):
            layer._base_weight_loader(layer.weight, w, name)
    else:
        layer = ref_layers.LoRAMergedColumnParallelLinear(
            case["in_f"], case["outs"], bias=False, lora_targets=case["targets"], max_loras=S, max_lora_rank=r
        )
        for i, w in enumerate(inputs["weights"]):
            layer._base_weight_loader(layer.weight, w, i)
    payload = cases.shard_payload(case, inputs, tp_rank)
    targets = inputs["targets"]
    with torch.no_grad():
        for slot, ad in payload.items():
            if kind in ("linear", "row"):
                layer.set_slot_lora(slot, ad["a"][targets[0]], ad["b"][targets[0]], ad["rank"], ad["scaling"])
            else:
                layer.set_slot_lora(
                    slot, torch.stack([ad["a"][t] for t in targets]), [ad["b"][t] for t in targets], ad["rank"],
                    ad["scaling"],
                )
    x = inputs["x"]
    if kind == "row" and tp > 1:
        x = x.chunk(tp, 1)[tp_rank]
    ref_context.set_lora_context(ref_context.build_lora_context_from_token_to_slot(inputs["slots"]))
    with torch.no_grad():
        y = layer(x)
    ref_context.reset_lora_context()
    return y.detach().clone()


def main() -> None:
    torch.manual_seed(0)
    ref_lora.set_backend_for_testing(_reference_test_backend())
    out = {}

    # ---- layer cases ---------------------------------------------------------
    for case in cases.LAYER_CASES:
        inputs = cases.build_inputs(case)
        out[f"{case['name']}/insum"] = checksum(inputs["x"], *inputs["weights"])
        for rank in range(case.get("tp", 1)):
            out[f"{case['name']}/y_rank{rank}"] = run_reference_layer(case, inputs, rank).numpy()
    np.savez_compressed(os.path.join(HERE, "layers.npz"), **out)

    # ---- config 1: the CPU reference op of the benchmark definition ----------
    p = workloads.config1(0)
    ref_layers._get_world_size = lambda: 1
    ref_layers._get_rank = lambda: 0
    layer = ref_layers.LoRALinear(1024, 1024, bias=False, max_loras=4, max_lora_rank=16)
    layer.weight.data.copy_(p.weight.float())
    with torch.no_grad():
        # workloads folds scaling=2.0 into B already; hand the reference the same slab
        # values (scaling 1.0) so both sides multiply identical bf16-rounded numbers.
        for s in range(4):
            layer.set_slot_lora(s, p.a_slabs[0][s].float(), p.b_slabs[0][s].float(), 16, 1.0)
    ref_context.set_lora_context(ref_context.build_lora_context_from_token_to_slot(p.token_to_slot))
    with torch.no_grad():
        y = layer(p.x.float())
    ref_context.reset_lora_context()
    base = p.x.float() @ p.weight.float().T
    np.savez_compressed(
        os.path.join(HERE, "config1.npz"), y=y.numpy(), base=base.numpy(), slots=p.token_to_slot.numpy(),
        insum=checksum(p.x.float(), p.weight.float(), p.a_slabs[0].float(), p.b_slabs[0].float()),
    )

    # ---- metadata ----------------------------------------------------------------
    from nanovllm_voxcpm.engine.model_runner import BaseModelRunner

    meta = {}
    for i, (max_loras, slots) in enumerate(cases.METADATA_CASES):
        plan = ref_manager.build_lora_batch_plan_from_token_to_slot({}, list(slots))
        meta[f"{i}/plan_sorted"] = np.asarray(plan.token_indices_sorted_by_slot, dtype=np.int32)
        meta[f"{i}/plan_active"] = np.asarray(plan.active_slot_ids, dtype=np.int32)
        meta[f"{i}/plan_counts"] = np.asarray(plan.num_tokens_per_slot, dtype=np.int32)
        meta[f"{i}/plan_offsets"] = np.asarray(plan.slot_start_offsets, dtype=np.int32)
        tts = torch.tensor(slots, dtype=torch.int32)
        ctx = ref_context.build_lora_context_from_token_to_slot(tts)
        meta[f"{i}/ctx_no_lora"] = np.asarray([int(ctx.no_lora_flag), ctx.num_active_loras], dtype=np.int32)
        for key in ("token_indices_sorted_by_slot", "active_slot_ids", "num_tokens_per_slot", "slot_start_offsets"):
            val = getattr(ctx, key)
            meta[f"{i}/ctx_{key}"] = np.zeros(0, np.int32) if val is None else val.numpy().astype(np.int32)
        if len(slots):
            km = LoRAKernelMeta.make(max_loras=max_loras, max_num_tokens=len(slots), device="cpu")
            km.prepare_tensors(tts)
            meta[f"{i}/vllm_flags"] = np.asarray([int(km.no_lora_flag), km.num_active_loras], dtype=np.int32)
            if not km.no_lora_flag:
                meta[f"{i}/vllm_sorted"] = km.token_indices_sorted_by_lora_ids.numpy().copy()
            meta[f"{i}/vllm_ids"] = km.active_lora_ids.numpy().copy()
            meta[f"{i}/vllm_counts"] = km.num_tokens_per_lora.numpy().copy()
            meta[f"{i}/vllm_starts"] = km.lora_token_start_loc.numpy().copy()
        # CUDA-graph buffers (CPU tensors stand in for the device buffers)
        max_rows = max(len(slots), 1) + 3
        bufs = BaseModelRunner._make_graph_domain_buffers(None, max_rows, max_loras + 1)
        graph_vars = {"lora_domains": {"lm_domain": bufs}}
        gctx = ref_manager.build_lora_context_from_batch_plan.__globals__["LoRAContext"](
            token_to_slot=tts,
            token_indices_sorted_by_slot=torch.tensor(plan.token_indices_sorted_by_slot, dtype=torch.int32),
            active_slot_ids=torch.tensor(plan.active_slot_ids, dtype=torch.int32),
            num_tokens_per_slot=torch.tensor(plan.num_tokens_per_slot, dtype=torch.int32),
            slot_start_offsets=torch.tensor(plan.slot_start_offsets, dtype=torch.int32),
            no_lora_flag=not plan.active_slot_ids,
            num_active_loras=len(plan.active_slot_ids),
        )
        if plan.active_slot_ids:
            BaseModelRunner._copy_lora_domain_to_graph_vars(None, graph_vars, "lm_domain", gctx)
            for key, val in bufs.items():
                meta[f"{i}/graph_{key}"] = val.numpy().copy()
    np.savez_compressed(os.path.join(HERE, "metadata.npz"), **meta)
    ref_lora.set_backend_for_testing(None)
    print("wrote", [f for f in os.listdir(HERE) if f.endswith(".npz")])


if __name__ == "__main__":
    main()
