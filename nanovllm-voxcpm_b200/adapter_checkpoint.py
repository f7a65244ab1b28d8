"""LoRA adapter checkpoints: the on-disk format in, slot payloads (per tensor-parallel rank) out.

Format (the reference's, ``nanovllm_voxcpm/models/voxcpm2/lora_loader.py:13-14,55-93,132-169``; the v1
loader ``models/voxcpm/lora_loader.py`` behaves the same): a directory with

* ``lora_weights.safetensors`` - tensors named ``<module path>.lora_A`` ``[rank, in]`` and
  ``<module path>.lora_B`` ``[out, rank]``; any run of the prefixes ``base_model.model.``, ``model.``,
  ``module.`` is dropped; a ``.lora_A.weight`` / ``.lora_B.weight`` suffix is refused; other keys are
  ignored. ``q_proj / k_proj / v_proj`` fold into the packed ``qkv_proj`` module (slices in q, k, v
  order), ``gate_proj / up_proj`` into ``gate_up_proj`` (``models/voxcpm2/model.py:491-497``);
* ``lora_config.json`` - ``{"lora_config": {"r" | "rank": int, "alpha" | "lora_alpha": float}}``; the
  rank may be left out (taken from the tensors), alpha may not; ``scaling = alpha / rank``.

Payloads come out as fp32 (the reference converts on load, ``lora_loader.py:114``; the slab dtype
is applied when a slot is written). Tensor-parallel sharding follows ``lora_loader.py:235-263``:
column-parallel packed modules split every ``lora_B`` on the output dim, row-parallel ``o_proj`` /
``down_proj`` split ``lora_A`` on the input dim and keep ``lora_B`` whole; anything else is replicated.
``row_parallel_lora_b="output_sharded"`` additionally splits the row-parallel ``lora_B`` on the output
dim, which is what ``LoRARowParallelLinear(lora_tp_mode="allreduce_tmp" | "peer_exchange")`` holds.

Unlike the reference, which materialises the whole adapter and then every rank's copies, a rank's
payload is read shard by shard straight into ONE host arena (pinned when CUDA is present), so that
admission (``slot_loader.SlotLoader``) can move it with a single host-to-device copy and no repacking;
``tp_rank=`` loads one rank's shard only (one process per GPU needs no more).
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path

import torch

WEIGHTS_FILE = "lora_weights.safetensors"
CONFIG_FILE = "lora_config.json"

#: projection leaf -> (packed module, slice key); ``models/voxcpm2/model.py:491-497``
PACKED_MODULES_MAPPING = {
    "q_proj": ("qkv_proj", "q"),
    "k_proj": ("qkv_proj", "k"),
    "v_proj": ("qkv_proj", "v"),
    "gate_proj": ("gate_up_proj", 0),
    "up_proj": ("gate_up_proj", 1),
}
_QKV_ORDER = {"q": 0, "k": 1, "v": 2}
_DROPPED_PREFIXES = ("base_model.model.", "model.", "module.")
_ARENA_ALIGN = 64


@dataclass
class LoRAModulePayload:
    """What a layer's ``set_slot_lora`` takes (``engine/lora_manager.py:25-30``)."""

    lora_a: torch.Tensor
    lora_b: torch.Tensor | list[torch.Tensor]
    effective_rank: int
    scaling: float


@dataclass
class LoRAModelPayload:
    """One adapter for one rank (``engine/lora_manager.py:33-37``); ``arena`` is the single host buffer
    every tensor of ``modules`` is a view of (``None`` for payloads assembled by hand)."""

    modules: dict[str, LoRAModulePayload]
    rank: int
    alpha: float
    arena: torch.Tensor | None = field(default=None, repr=False, compare=False)


# --------------------------------------------------------------------------------------------- names
def _strip_prefixes(name: str) -> str:
    while True:
        for prefix in _DROPPED_PREFIXES:
            if name.startswith(prefix):
                name = name[len(prefix):]
                break
        else:
            return name


def parse_weight_key(key: str, packed_modules_mapping=PACKED_MODULES_MAPPING):
    """``(module name, kind, slice key, "a" | "b")`` of a checkpoint key, ``None`` for keys that are not
    adapter weights. Kinds: ``qkv``, ``merged_column``, ``row_parallel``, ``linear``."""
    if key.endswith((".lora_A.weight", ".lora_B.weight")):
        raise ValueError("Unsupported LoRA tensor suffix; expected keys ending in '.lora_A' or '.lora_B'")
    if key.endswith(".lora_A"):
        which = "a"
    elif key.endswith(".lora_B"):
        which = "b"
    else:
        return None
    path = _strip_prefixes(key[: -len(".lora_A")])
    parent, _, leaf = path.rpartition(".")
    packed = packed_modules_mapping.get(leaf)
    if packed is not None:
        module, target = packed
        kind = "qkv" if isinstance(target, str) else "merged_column"
        return (f"{parent}.{module}" if parent else module), kind, target, which
    if leaf in ("o_proj", "down_proj"):
        return path, "row_parallel", leaf, which
    return path, "linear", leaf, which


# --------------------------------------------------------------------------------------------- config
def read_adapter_config(checkpoint_dir: Path) -> dict:
    with (checkpoint_dir / CONFIG_FILE).open("r", encoding="utf-8") as f:
        raw = json.load(f)
    if not isinstance(raw, dict):
        raise ValueError("LoRA config must be a JSON object")
    cfg = raw.get("lora_config")
    if not isinstance(cfg, dict):
        raise ValueError("lora_config.json must contain a 'lora_config' object")
    return cfg


def _alpha_of(cfg: dict) -> float:
    alpha = cfg.get("alpha", cfg.get("lora_alpha"))
    if alpha is None:
        raise ValueError("LoRA config must define alpha or lora_alpha")
    alpha = float(alpha)
    if alpha <= 0:
        raise ValueError(f"LoRA alpha must be > 0, got {alpha}")
    return alpha


def _rank_of(cfg: dict, ranks_seen: set[int]) -> int:
    if not ranks_seen:
        raise ValueError("LoRA checkpoint does not contain any LoRA A tensors")
    if len(ranks_seen) != 1:
        raise ValueError(f"LoRA checkpoint contains inconsistent ranks: {sorted(ranks_seen)}")
    (inferred,) = ranks_seen
    declared = cfg.get("r", cfg.get("rank"))
    if declared is None:
        return inferred
    declared = int(declared)
    if declared <= 0:
        raise ValueError(f"LoRA rank must be > 0, got {declared}")
    if declared != inferred:
        raise ValueError(f"LoRA config rank {declared} does not match tensor rank {inferred}")
    return declared


# --------------------------------------------------------------------------------------------- index
@dataclass
class _Module:
    name: str
    kind: str
    targets: list = field(default_factory=list)        # in order of first appearance
    a_keys: dict = field(default_factory=dict)         # target -> checkpoint key
    b_keys: dict = field(default_factory=dict)

    def ordered_targets(self) -> list:
        if self.kind == "qkv":
            return sorted(self.targets, key=lambda t: _QKV_ORDER[str(t)])
        if self.kind == "merged_column":
            return sorted(self.targets, key=int)
        return self.targets


def _index(keys, packed_modules_mapping) -> dict[str, _Module]:
    modules: dict[str, _Module] = {}
    for key in keys:
        parsed = parse_weight_key(key, packed_modules_mapping)
        if parsed is None:
            continue
        name, kind, target, which = parsed
        module = modules.setdefault(name, _Module(name, kind))
        if target not in module.targets:
            module.targets.append(target)
        (module.a_keys if which == "a" else module.b_keys)[target] = key
    for module in modules.values():
        missing_a = [t for t in module.targets if t not in module.a_keys]
        missing_b = [t for t in module.targets if t not in module.b_keys]
        if missing_a or missing_b:
            raise ValueError(
                f"Incomplete LoRA tensors for module '{module.name}': missing_a={missing_a}, missing_b={missing_b}")
    return modules


# --------------------------------------------------------------------------------------------- shards
def _chunk(n: int, tp_rank: int, tp_size: int) -> tuple[int, int]:
    """(start, length) of ``torch.chunk(tp_size)[tp_rank]`` along a dim of ``n``."""
    if tp_size <= 1:
        return 0, n
    step = math.ceil(n / tp_size)
    start = tp_rank * step
    if start >= n:
        raise ValueError(f"a dim of {n} cannot be split over {tp_size} ranks")
    return start, min(step, n - start)


def _shard_rule(module: _Module, row_parallel_lora_b: str) -> tuple[bool, bool]:
    """(split lora_A on its input dim, split lora_B on its output dim) under tensor parallelism."""
    if module.name.endswith(("qkv_proj", "gate_up_proj")):
        return False, True
    if module.name.endswith(("o_proj", "down_proj")):
        return True, row_parallel_lora_b == "output_sharded"
    return False, False


class _Arena:
    def __init__(self, nbytes: int, pin: bool):
        self.buffer = torch.empty(max(nbytes, _ARENA_ALIGN), dtype=torch.uint8, pin_memory=pin)
        self.cursor = 0

    @staticmethod
    def span(shape) -> int:
        return (4 * math.prod(shape) + _ARENA_ALIGN - 1) // _ARENA_ALIGN * _ARENA_ALIGN

    def take(self, shape) -> torch.Tensor:
        nbytes = 4 * math.prod(shape)
        view = self.buffer[self.cursor: self.cursor + nbytes].view(torch.float32).view(*shape)
        self.cursor += self.span(shape)
        return view


def _rank_payload(f, modules, shapes, rank, alpha, tp_rank, tp_size, row_parallel_lora_b, pin) -> LoRAModelPayload:
    plan = []  # (module, targets, a shape, [(b shape)], a cols, b rows)
    total = 0
    for module in modules.values():
        targets = module.ordered_targets()
        split_a, split_b = _shard_rule(module, row_parallel_lora_b) if tp_size > 1 else (False, False)
        a_shapes = {tuple(shapes[module.a_keys[t]]) for t in targets}
        if len(a_shapes) != 1:
            raise ValueError(f"LoRA A tensors of module '{module.name}' differ in shape: {sorted(a_shapes)}")
        (a_shape,) = a_shapes
        a_cols = _chunk(a_shape[1], tp_rank, tp_size) if split_a else (0, a_shape[1])
        b_rows = [(_chunk(shapes[module.b_keys[t]][0], tp_rank, tp_size) if split_b
                   else (0, shapes[module.b_keys[t]][0])) for t in targets]
        packed = module.kind in ("qkv", "merged_column")
        a_out = (len(targets), a_shape[0], a_cols[1]) if packed else (a_shape[0], a_cols[1])
        b_out = [(rows[1], shapes[module.b_keys[t]][1]) for t, rows in zip(targets, b_rows)]
        total += _Arena.span(a_out) + sum(_Arena.span(s) for s in b_out)
        plan.append((module, targets, packed, a_out, b_out, a_cols, b_rows))

    arena = _Arena(total, pin)
    out: dict[str, LoRAModulePayload] = {}
    scaling = alpha / rank
    for module, targets, packed, a_out, b_out, a_cols, b_rows in plan:
        lora_a = arena.take(a_out)
        for i, t in enumerate(targets):
            src = f.get_slice(module.a_keys[t])[:, a_cols[0]: a_cols[0] + a_cols[1]]
            (lora_a[i] if packed else lora_a).copy_(src)  # converts to fp32
        lora_b = []
        for t, shape, rows in zip(targets, b_out, b_rows):
            dst = arena.take(shape)
            dst.copy_(f.get_slice(module.b_keys[t])[rows[0]: rows[0] + rows[1], :])
            lora_b.append(dst)
        out[module.name] = LoRAModulePayload(lora_a=lora_a, lora_b=lora_b if packed else lora_b[0],
                                             effective_rank=rank, scaling=scaling)
    return LoRAModelPayload(modules=out, rank=rank, alpha=alpha, arena=arena.buffer)


# --------------------------------------------------------------------------------------------- API
def load_lora_checkpoint(path: str, *, tp_size: int = 1, tp_rank: int | None = None,
                         row_parallel_lora_b: str = "replicated",
                         packed_modules_mapping=PACKED_MODULES_MAPPING, pin_memory: bool | None = None):
    """The adapter at ``path`` as slot payloads.

    ``tp_size <= 1``: one ``LoRAModelPayload``. ``tp_size > 1``: the list of all ranks' payloads (the
    reference's return value), or only rank ``tp_rank``'s when that is given.
    """
    from safetensors import safe_open

    if row_parallel_lora_b not in ("replicated", "output_sharded"):
        raise ValueError(f"unknown row_parallel_lora_b {row_parallel_lora_b!r}")
    checkpoint_dir = Path(path)
    if not checkpoint_dir.is_dir():
        raise FileNotFoundError(f"LoRA checkpoint directory not found: {checkpoint_dir}")
    if not (checkpoint_dir / WEIGHTS_FILE).is_file():
        raise FileNotFoundError(f"Missing LoRA weights file: {checkpoint_dir / WEIGHTS_FILE}")
    if not (checkpoint_dir / CONFIG_FILE).is_file():
        raise FileNotFoundError(f"Missing LoRA config file: {checkpoint_dir / CONFIG_FILE}")
    cfg = read_adapter_config(checkpoint_dir)
    alpha = _alpha_of(cfg)
    pin = torch.cuda.is_available() if pin_memory is None else pin_memory
    tp_size = max(int(tp_size), 1)
    if tp_rank is not None and not 0 <= tp_rank < tp_size:
        raise ValueError(f"tp_rank {tp_rank} outside 0..{tp_size - 1}")

    with safe_open(checkpoint_dir / WEIGHTS_FILE, framework="pt", device="cpu") as f:
        modules = _index(f.keys(), packed_modules_mapping)
        if not modules:
            raise ValueError("LoRA checkpoint does not contain any supported module weights")
        shapes = {key: tuple(f.get_slice(key).get_shape())
                  for m in modules.values() for key in (*m.a_keys.values(), *m.b_keys.values())}
        rank = _rank_of(cfg, {shapes[key][0] for m in modules.values() for key in m.a_keys.values()})
        build = lambda r: _rank_payload(f, modules, shapes, rank, alpha, r, tp_size, row_parallel_lora_b, pin)  # noqa: E731
        if tp_size == 1:
            return build(0)
        if tp_rank is not None:
            return build(tp_rank)
        return [build(r) for r in range(tp_size)]


def load_voxcpm2_lora_checkpoint(path: str, *, tp_size: int = 1):
    """The reference's entry point (``models/voxcpm2/lora_loader.py:27-41``)."""
    return load_lora_checkpoint(path, tp_size=tp_size)


def load_voxcpm_lora_checkpoint(path: str, *, tp_size: int = 1):
    """The reference's entry point of the v1 model (``models/voxcpm/lora_loader.py``)."""
    return load_lora_checkpoint(path, tp_size=tp_size)


def save_lora_checkpoint(path: str, tensors: dict[str, torch.Tensor], *, rank: int | None, alpha: float) -> Path:
    """Writes ``tensors`` (``<module path>.lora_A`` / ``.lora_B``) and the config in the format read above."""
    from safetensors.torch import save_file

    checkpoint_dir = Path(path)
    checkpoint_dir.mkdir(parents=True, exist_ok=True)
    save_file({k: v.detach().cpu().contiguous() for k, v in tensors.items()}, str(checkpoint_dir / WEIGHTS_FILE))
    cfg = {"alpha": float(alpha)}
    if rank is not None:
        cfg["r"] = int(rank)
    (checkpoint_dir / CONFIG_FILE).write_text(json.dumps({"lora_config": cfg}), encoding="utf-8")
    return checkpoint_dir
