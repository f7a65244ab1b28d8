"""Seeded inputs shared by make_glue_golden.py (reference modules) and tests/test_glue_oracle.py (oracle)."""

import torch

T, HIDDEN, INTER, HEADS, KV_HEADS, HEAD_DIM, MAX_POS = 12, 256, 384, 4, 2, 64, 512
EPS = 1e-6
ROPE = dict(base=10000.0, short_factor=[1.0 + 0.01 * i for i in range(HEAD_DIM // 2)],
            long_factor=[2.0 + 0.05 * i for i in range(HEAD_DIM // 2)], original_max_position=128)


def inputs(dtype: torch.dtype):
    gen = torch.Generator().manual_seed(1234)
    x = (torch.randn(T, HIDDEN, generator=gen) * 1.5).to(dtype)
    residual = (torch.randn(T, HIDDEN, generator=gen) * 3.0).to(dtype)
    weight = (1.0 + 0.1 * torch.randn(HIDDEN, generator=gen)).to(dtype)
    gate_up = (torch.randn(T, 2 * INTER, generator=gen) * 2.0).to(dtype)
    q = torch.randn(T, HEADS * HEAD_DIM, generator=gen).to(dtype)
    k = torch.randn(T, KV_HEADS * HEAD_DIM, generator=gen).to(dtype)
    positions = torch.randint(0, MAX_POS, (T,), generator=gen)
    return dict(x=x, residual=residual, weight=weight, gate_up=gate_up, q=q, k=k, positions=positions)
