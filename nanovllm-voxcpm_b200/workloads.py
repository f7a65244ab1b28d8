"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (no dataset or checkpoint is involved: weights are random-init).

All tensors are drawn from a CPU ``torch.Generator`` so that a CPU checker and the GPU
see identical bits; move them with ``to_device``.

Configurations (sizes per projection are ``in -> [slice widths]``):
  * ``config1``: one plain linear 1024 -> 1024, T=64, 4 adapters rank 16, scaling 2.0,
    slots uniform over {0..3} with 25 % set to -1, x~N(0,1), W/A/B~N(0,0.02), seed 0.
  * ``DECODE_LAYER`` (decode BGMV): 256 sequences x 1 token, hidden 1024, 16 q / 2 kv
    heads x 64, intermediate 4096, 32 adapters rank 32, 10 % of rows without adapter.
  * ``PREFILL_LAYER`` (prefill SGMV): 16 requests of 64..1024 tokens (<= 8192 total),
    hidden 2048, intermediate 6144, 16 adapters with ranks cycling 8,16,64 in a rank-64
    slab, one adapter per request; qkv widths 2048/256/256 (16 q + 2 kv heads x 128).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

DECODE_LAYER = {
    "qkv": (1024, [1024, 128, 128]),
    "o": (1024, [1024]),
    "gate_up": (1024, [4096, 4096]),
    "down": (4096, [1024]),
}
PREFILL_LAYER = {
    "qkv": (2048, [2048, 256, 256]),
    "o": (2048, [2048]),
    "gate_up": (2048, [6144, 6144]),
    "down": (6144, [2048]),
}


@dataclass
class Projection:
    """Inputs of one multi-LoRA linear call (slab layout of the layers)."""

    x: torch.Tensor  # [T, in]
    y: torch.Tensor  # [T, sum(out)]   base output the delta is added to
    a_slabs: list[torch.Tensor]  # n x [S, r_max, in]
    b_slabs: list[torch.Tensor]  # n x [S, out_s, r_max]   (scaling folded in)
    out_sizes: list[int]
    col_offsets: list[int]
    ranks: torch.Tensor  # int32 [S] effective rank per slot
    token_to_slot: torch.Tensor  # int32 [T]
    weight: torch.Tensor | None = None  # [sum(out), in] base weight when generated
    extras: dict = field(default_factory=dict)

    def to_device(self, device) -> "Projection":
        mv = lambda t: None if t is None else t.to(device)  # noqa: E731
        return Projection(
            mv(self.x), mv(self.y), [mv(a) for a in self.a_slabs], [mv(b) for b in self.b_slabs],
            list(self.out_sizes), list(self.col_offsets), mv(self.ranks), mv(self.token_to_slot), mv(self.weight),
            dict(self.extras),
        )


def _randn(gen, *shape, std=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, generator=gen, dtype=torch.float32) * std).to(dtype)


def make_slabs(gen, S, r_max, in_dim, out_sizes, ranks, dtype=torch.bfloat16, scaling=1.0, std=0.02):
    """Zero-padded slabs: slot s holds a rank-``ranks[s]`` adapter, B pre-scaled."""
    a_slabs, b_slabs = [], []
    for out in out_sizes:
        a = torch.zeros(S, r_max, in_dim, dtype=dtype)
        b = torch.zeros(S, out, r_max, dtype=dtype)
        for s in range(S):
            r = int(ranks[s])
            a[s, :r] = _randn(gen, r, in_dim, std=std, dtype=dtype)
            b[s, :, :r] = (_randn(gen, out, r, std=std, dtype=torch.float32) * scaling).to(dtype)
        a_slabs.append(a)
        b_slabs.append(b)
    return a_slabs, b_slabs


def uniform_slots(gen, T, S, p_none):
    slots = torch.randint(0, S, (T,), generator=gen, dtype=torch.int32)
    drop = torch.rand(T, generator=gen) < p_none
    return torch.where(drop, torch.full_like(slots, -1), slots)


def make_projection(
    seed, T, in_dim, out_sizes, S, r_max, *, ranks=None, p_none=0.1, token_to_slot=None, dtype=torch.bfloat16,
    scaling=1.0, with_weight=False, y_std=1.0,
) -> Projection:
    gen = torch.Generator().manual_seed(seed)
    ranks_t = torch.full((S,), r_max, dtype=torch.int32) if ranks is None else torch.as_tensor(ranks, dtype=torch.int32)
    x = _randn(gen, T, in_dim, dtype=dtype)
    weight = _randn(gen, sum(out_sizes), in_dim, std=0.02, dtype=dtype) if with_weight else None
    a_slabs, b_slabs = make_slabs(gen, S, r_max, in_dim, out_sizes, ranks_t.tolist(), dtype, scaling)
    if token_to_slot is None:
        token_to_slot = uniform_slots(gen, T, S, p_none)
    if with_weight:
        y = (x.float() @ weight.float().T).to(dtype)
    else:
        y = _randn(gen, T, sum(out_sizes), std=y_std, dtype=dtype)
    cols, pos = [], 0
    for w in out_sizes:
        cols.append(pos)
        pos += w
    return Projection(x, y, a_slabs, b_slabs, list(out_sizes), cols, ranks_t,
                      torch.as_tensor(token_to_slot, dtype=torch.int32), weight)


def config1(seed: int = 0) -> Projection:
    """CPU reference op of the benchmark definition (scaling 2.0 folded into B)."""
    return make_projection(seed, 64, 1024, [1024], 4, 16, p_none=0.25, scaling=2.0, with_weight=True)


def decode_projection(name: str, seed: int = 0, T: int = 256, S: int = 32, r: int = 32, p_none: float = 0.1):
    in_dim, outs = DECODE_LAYER[name]
    return make_projection(seed, T, in_dim, outs, S, r, p_none=p_none)


def prefill_lengths(seed: int = 0, n_req: int = 16, lo: int = 64, hi: int = 1024, cap: int = 8192) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (n_req,), generator=gen).tolist()
    while sum(lens) > cap:  # trim the longest request until the pack fits
        i = max(range(n_req), key=lambda k: lens[k])
        lens[i] = max(lo, lens[i] - (sum(lens) - cap))
    return lens


def prefill_projection(name: str, seed: int = 0, lengths=None, S: int = 16, r_max: int = 64):
    in_dim, outs = PREFILL_LAYER[name]
    lengths = lengths or prefill_lengths(seed)
    ranks = [(8, 16, 64)[s % 3] for s in range(S)]
    slots = []
    for req, n in enumerate(lengths):
        slots.extend([req % S] * n)
    p = make_projection(seed + 1, sum(lengths), in_dim, outs, S, r_max, ranks=ranks, token_to_slot=slots)
    p.extras["lengths"] = lengths
    return p


def algorithmic_bytes(p: Projection, elem: int = 2) -> int:
    """Bytes one launch must move: each active slot's A rows (effective rank) and B
    slab once, x rows and a read+write of y for rows that carry an adapter."""
    tts = p.token_to_slot
    active = torch.unique(tts[tts >= 0]).tolist()
    t_lora = int((tts >= 0).sum())
    in_dim = p.x.shape[1]
    n = len(p.out_sizes)
    r_max = p.a_slabs[0].shape[1]
    total = 0
    for s in active:
        r = min(int(p.ranks[s]), r_max)
        total += n * r * in_dim * elem  # lora_A rows that hold data
        total += sum(p.out_sizes) * r * elem  # lora_B columns that hold data
    total += t_lora * in_dim * elem
    total += 2 * t_lora * sum(p.out_sizes) * elem
    return total
