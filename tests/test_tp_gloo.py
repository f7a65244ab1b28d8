"""Tensor-parallel host logic with two real ranks on the CPU (gloo): sharding of the slabs,
the row-parallel exchange in both modes and the single `[T, out]` / `[T, r]` all-reduce.
The kernels are replaced by the CPU oracle (the product has no CPU path); what is tested is
everything around them."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_ops():
    """shrink_into / expand_into stand-ins with the C-ABI semantics, on the CPU oracle."""
    from oracle import lora_oracle as O

    def shrink_into(out, x, a_slabs, token_to_slot, scaling):
        out.copy_(O.shrink(x, a_slabs, token_to_slot, scaling).to(out.dtype))

    def expand_into(y, tmp, b_slabs, token_to_slot, *, offset_start, add_inputs):
        y.copy_(O.expand(y, tmp, b_slabs, token_to_slot, offset_start, add_inputs).to(y.dtype))

    return shrink_into, expand_into


def _worker(rank: int, world: int, port: int, results):
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for p in (root, os.path.join(root, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from helpers import OracleBackend
    from nanovllm_voxcpm_b200 import context as CTX
    from nanovllm_voxcpm_b200 import layers as L
    from nanovllm_voxcpm_b200 import lora as LORA
    from nanovllm_voxcpm_b200 import lora_ops
    from oracle import lora_oracle as O

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        LORA.set_backend_for_testing(OracleBackend())
        lora_ops.shrink_into, lora_ops.expand_into = _oracle_ops()
        g = torch.Generator().manual_seed(7)  # same tensors on every rank
        T, hidden, out_f, S, r = 12, 32, 24, 3, 4
        x = torch.randn(T, hidden, generator=g)
        w = torch.randn(out_f, hidden, generator=g) * 0.1
        bias = torch.randn(out_f, generator=g) * 0.1
        slots = torch.tensor([0, 2, -1, 1, 1, 0, -1, 2, 2, 0, 1, -1], dtype=torch.int32)
        adapters = {s: (torch.randn(r, hidden, generator=g) * 0.2, torch.randn(out_f, r, generator=g) * 0.2, 1.0 + s)
                    for s in range(S)}
        # single-process truth from the oracle
        a_full, b_full = torch.zeros(S, r, hidden), torch.zeros(S, out_f, r)
        for s, (a, b, sc) in adapters.items():
            O.write_slot(a_full, b_full, s, a, b, r, sc)
        want = O.linear_lora(x, w, bias, [a_full], [b_full], [0], slots)

        CTX.set_lora_context(CTX.build_lora_context_from_token_to_slot(slots))
        x_shard = x.chunk(world, 1)[rank]
        for mode in ("partial_y", "allreduce_tmp"):
            layer = L.LoRARowParallelLinear(hidden, out_f, bias=True, max_loras=S, max_lora_rank=r, lora_tp_mode=mode)
            assert layer.tp_size == world and layer.tp_rank == rank
            layer.load_base_shard(w)
            layer.bias.data.copy_(bias)
            for s, (a, b, sc) in adapters.items():
                a_shard = a.chunk(world, 1)[rank]
                b_shard = b if mode == "partial_y" else b.chunk(world, 0)[rank]
                layer.validate_slot_lora_payload(a_shard, b_shard, r, sc)
                layer.set_slot_lora(s, a_shard, b_shard, r, sc)
            with torch.no_grad():
                y = layer(x_shard)
            torch.testing.assert_close(y, want, atol=1e-4, rtol=1e-4, msg=f"row-parallel mode {mode}")
            assert layer.lora_B.shape[1] == (out_f if mode == "partial_y" else out_f // world)

        # column-parallel: lora_B sharded on the output dim, no collective; gather and compare
        col = L.LoRAMergedColumnParallelLinear(hidden, [out_f, out_f], max_loras=S, max_lora_rank=r)
        w2 = [w, w * 0.5]
        for i, wi in enumerate(w2):
            col.load_base_shard(wi, i)
        for s, (a, b, sc) in adapters.items():
            col.set_slot_lora(s, torch.stack([a, a]), [b.chunk(world, 0)[rank], (b * 2).chunk(world, 0)[rank]], r, sc)
        with torch.no_grad():
            y_col = col(x)
        parts = [torch.empty_like(y_col) for _ in range(world)]
        dist.all_gather(parts, y_col)
        half = out_f // world
        gate = torch.cat([p[:, :half] for p in parts], 1)
        up = torch.cat([p[:, half:] for p in parts], 1)
        b2_full = torch.zeros(S, out_f, r)
        a2_full = torch.zeros(S, r, hidden)
        for s, (a, b, sc) in adapters.items():
            O.write_slot(a2_full, b2_full, s, a, b * 2, r, sc)
        torch.testing.assert_close(gate, O.linear_lora(x, w2[0], None, [a_full], [b_full], [0], slots), atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(up, O.linear_lora(x, w2[1], None, [a2_full], [b2_full], [0], slots), atol=1e-4, rtol=1e-4)
        results[rank] = "ok"
    except Exception as exc:  # surfaced by the parent
        results[rank] = f"{type(exc).__name__}: {exc}"
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_rank_tensor_parallel_lora_layers():
    world = 2
    port = _free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}, dict(results)
