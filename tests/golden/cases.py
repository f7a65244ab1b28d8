"""Seeded case definitions shared by the golden-vector generator (which runs the
reference) and by the tests (which run the oracle and the CUDA path on the same inputs).

A layer case is a dict: kind, constructor sizes, tp size, adapters per slot
(rank, scaling), token->slot map, seed.  ``build_inputs`` turns it into tensors.
"""

from __future__ import annotations

import torch

LAYER_CASES = [
    dict(name="linear_bias", kind="linear", in_f=96, out_f=64, bias=True, S=3, r_max=16,
         adapters={0: (16, 1.0), 2: (4, 0.5)}, slots=[0, -1, 2, 2, 0, -1, 1, 0, 2, -1, 0, 2], seed=11),
    dict(name="qkv_tp1", kind="qkv", hidden=64, head=16, heads=4, kv_heads=2, targets=None, tp=1, S=3, r_max=8,
         adapters={0: (8, 1.0), 1: (2, 2.0), 2: (5, 0.25)}, slots=[2, 0, 1, -1, 0, 0, 2, -1, 1, 1], seed=12),
    dict(name="qkv_tp2", kind="qkv", hidden=64, head=16, heads=4, kv_heads=2, targets=None, tp=2, S=3, r_max=8,
         adapters={0: (8, 1.0), 1: (2, 2.0), 2: (5, 0.25)}, slots=[2, 0, 1, -1, 0, 0, 2, -1, 1, 1], seed=13),
    dict(name="qkv_partial_qv", kind="qkv", hidden=64, head=16, heads=4, kv_heads=2, targets=["q", "v"], tp=1, S=2,
         r_max=8, adapters={0: (8, 1.0), 1: (3, 1.5)}, slots=[1, 0, -1, 1, 0, 0], seed=14),
    dict(name="merged_tp1", kind="merged", in_f=64, outs=[96, 96], targets=None, tp=1, S=4, r_max=16,
         adapters={0: (16, 1.0), 1: (8, 0.5), 3: (1, 4.0)}, slots=[3, 3, 0, -1, 1, 0, 2, 1, -1, 3, 0], seed=15),
    dict(name="merged_only_up", kind="merged", in_f=64, outs=[96, 96], targets=[1], tp=1, S=2, r_max=16,
         adapters={0: (16, 1.0), 1: (8, 0.5)}, slots=[1, 0, -1, 1], seed=16),
    dict(name="merged_tp2", kind="merged", in_f=64, outs=[96, 96], targets=None, tp=2, S=4, r_max=16,
         adapters={0: (16, 1.0), 1: (8, 0.5), 3: (1, 4.0)}, slots=[3, 3, 0, -1, 1, 0, 2, 1, -1, 3, 0], seed=17),
    dict(name="row_tp1", kind="row", in_f=128, out_f=64, bias=True, tp=1, S=3, r_max=8,
         adapters={0: (8, 1.0), 1: (4, 2.0)}, slots=[1, 0, -1, 2, 0, 1, 1], seed=18),
    dict(name="row_tp2", kind="row", in_f=128, out_f=64, bias=True, tp=2, S=3, r_max=8,
         adapters={0: (8, 1.0), 1: (4, 2.0)}, slots=[1, 0, -1, 2, 0, 1, 1], seed=19),
]

#: token->slot maps for the metadata fixtures (max_loras, map)
METADATA_CASES = [
    (2, [0, -1, 1]),
    (1, [0, 0, -1, 0]),
    (4, [-1, -1, -1]),
    (4, [3, 3, 3, 3]),
    (8, [5, 0, -1, 5, 7, 0, 0, -1, 2, 5, 7, 7, 1]),
    (3, []),
    (32, [(i * 7 + 3) % 32 if i % 9 else -1 for i in range(100)]),
]


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def build_inputs(case: dict) -> dict:
    """Full (un-sharded) tensors of a layer case, fp32."""
    g = _gen(case["seed"])
    kind = case["kind"]
    T = len(case["slots"])
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    if kind == "linear":
        in_f, outs, names = case["in_f"], [case["out_f"]], ["lin"]
    elif kind == "row":
        in_f, outs, names = case["in_f"], [case["out_f"]], ["row"]
    elif kind == "qkv":
        in_f = case["hidden"]
        outs = [case["heads"] * case["head"], case["kv_heads"] * case["head"], case["kv_heads"] * case["head"]]
        names = ["q", "k", "v"]
    else:
        in_f, outs, names = case["in_f"], list(case["outs"]), list(range(len(case["outs"])))
    x = rn(T, in_f)
    weights = [rn(o, in_f) * 0.1 for o in outs]
    bias = rn(sum(outs)) * 0.1 if case.get("bias") else None
    targets = case.get("targets") or names
    adapters = {}
    for slot, (rank, scaling) in case["adapters"].items():
        # payload tensors carry max rank rows; only the first `rank` are used
        a = {t: rn(case["r_max"], in_f) * 0.2 for t in targets}
        b = {t: rn(outs[names.index(t)], case["r_max"]) * 0.2 for t in targets}
        adapters[slot] = dict(rank=rank, scaling=scaling, a=a, b=b)
    return dict(x=x, weights=weights, bias=bias, names=names, outs=outs, targets=list(targets), adapters=adapters,
                slots=torch.tensor(case["slots"], dtype=torch.int32), in_f=in_f)


def shard_payload(case: dict, inputs: dict, tp_rank: int):
    """Per-rank adapter payloads following the reference loader's TP rule
    (models/voxcpm2/lora_loader.py:235-263): column-parallel layers shard lora_B rows,
    row-parallel layers shard lora_A columns."""
    tp = case.get("tp", 1)
    out = {}
    for slot, ad in inputs["adapters"].items():
        a, b = dict(ad["a"]), dict(ad["b"])
        if case["kind"] in ("qkv", "merged"):
            b = {t: v.chunk(tp, 0)[tp_rank] for t, v in b.items()}
        elif case["kind"] == "row":
            a = {t: v.chunk(tp, 1)[tp_rank] for t, v in a.items()}
        out[slot] = dict(rank=ad["rank"], scaling=ad["scaling"], a=a, b=b)
    return out
