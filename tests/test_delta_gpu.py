"""`lora_b200_delta` (the LoRA delta written, not added; -0.0 in rows without one) and the layers' LoRA-first
order built on it, against the oracle and against the add-after-GEMM order."""

import pytest
import torch

from nanovllm_voxcpm_b200 import _native as N
from nanovllm_voxcpm_b200 import context as CTX
from nanovllm_voxcpm_b200 import layers as L
from nanovllm_voxcpm_b200 import lora as LORA
from nanovllm_voxcpm_b200 import workloads as W
from oracle import lora_oracle as O

from helpers import assert_lora_close
from test_parity_gpu import DEV, metadata_for

pytestmark = pytest.mark.gpu
NEG_ZERO = -32768  # 0x8000 as int16


@pytest.fixture(autouse=True)
def _clean():
    CTX.reset_lora_context()
    for key in (N.OPT_CLUSTER, N.OPT_RING_KB):
        N.set_option(key, 0)
    N.set_option(N.OPT_PDL, 1)
    yield
    CTX.reset_lora_context()
    L.LORA_FIRST = False
    assert N.device_status() == 0


def run_delta(p: W.Projection, impl: int, convention: str, use_ranks=False, pad=0):
    d = p.to_device(DEV)
    S = d.a_slabs[0].shape[0]
    buf = torch.full((d.y.shape[0], d.y.shape[1] + pad), 7.0, dtype=d.y.dtype, device=DEV)
    y = buf[:, : d.y.shape[1]]
    LORA.launch_add(y, d.x, d.a_slabs, d.b_slabs, d.out_sizes, d.col_offsets, metadata_for(d.token_to_slot, convention, S),
                    1.0, rank_per_slot=d.ranks if use_ranks else None, impl=impl, overwrite=True)
    torch.cuda.synchronize()
    return buf.cpu()


def check_delta(p: W.Projection, buf: torch.Tensor, what: str, dead_slots=()):
    width = p.y.shape[1]
    out = buf[:, :width]
    assert bool((buf[:, width:] == 7.0).all()), f"{what}: columns beyond the row were written"
    want = O.add_lora(torch.zeros_like(p.y), p.x, p.a_slabs, p.b_slabs, p.token_to_slot, 1.0, p.col_offsets)
    assert_lora_close(out, want, what=what)
    none = p.token_to_slot < 0
    for s in dead_slots:
        none = none | (p.token_to_slot == s)
    covered = torch.zeros(width, dtype=torch.bool)
    for w, c in zip(p.out_sizes, p.col_offsets):
        covered[c: c + w] = True
    bits = out.view(torch.int16)
    assert bool((bits[none][:, covered] == NEG_ZERO).all()), f"{what}: rows without delta are not -0.0"
    assert bool((out[:, ~covered] == 7.0).all()), f"{what}: columns outside the slices were written"
    assert float(out[~none][:, covered].float().abs().max()) > 0


@pytest.mark.parametrize("convention", ["eager", "graph", "vllm"])
@pytest.mark.parametrize("name", ["qkv", "o", "gate_up", "down"])
def test_decode_delta_matches_oracle(name, convention):
    p = W.decode_projection(name, seed=11)
    for impl in (N.IMPL_AUTO, N.IMPL_BGMV):
        check_delta(p, run_delta(p, impl, convention), f"{name}/{convention}/{impl}")


@pytest.mark.parametrize("cluster", [1, 2, 8])
def test_delta_many_rows_per_bucket_idle_buckets_and_rank_zero(cluster):
    N.set_option(N.OPT_CLUSTER, cluster)
    # 200 rows over 3 of 8 slots (several 16-row passes per bucket, idle buckets do their share of the fill)
    p = W.decode_projection("gate_up", seed=5, T=200, S=8, p_none=0.3)
    gen = torch.Generator().manual_seed(1)
    used = torch.tensor([1, 4, 6])
    has = p.token_to_slot >= 0
    p.token_to_slot[has] = used[torch.randint(0, 3, (int(has.sum()),), generator=gen)].to(p.token_to_slot.dtype)
    check_delta(p, run_delta(p, N.IMPL_BGMV, "graph", pad=8), f"C{cluster}")
    # an adapter of rank 0 adds nothing: its rows are -0.0 too
    p.ranks = torch.full_like(p.ranks, p.a_slabs[0].shape[1])
    p.ranks[4] = 0
    for a in p.a_slabs:
        a[4].zero_()
    check_delta(p, run_delta(p, N.IMPL_BGMV, "graph", use_ranks=True), f"C{cluster}/rank0", dead_slots=(4,))


def test_delta_on_the_other_paths():
    """Shapes the fused decode kernel does not take: -0.0 fill, then the usual add (generic kernel; prefill kernels)."""
    p = W.make_projection(21, 33, 160, [48, 24], 3, 8, dtype=torch.float16, p_none=0.3)
    d = p.to_device(DEV)
    y = torch.full_like(d.y, 7.0)
    LORA.launch_add(y, d.x, d.a_slabs, d.b_slabs, d.out_sizes, d.col_offsets, metadata_for(d.token_to_slot, "eager", 3), 1.0,
                    overwrite=True)
    want = O.add_lora(torch.zeros_like(p.y), p.x, p.a_slabs, p.b_slabs, p.token_to_slot, 1.0, p.col_offsets)
    assert_lora_close(y.cpu(), want, what="fp16 generic")
    assert bool((y.cpu()[p.token_to_slot < 0].view(torch.int16) == NEG_ZERO).all())
    # slices that do not tile the output in 64-column units: fill, then the prefill kernels add
    p = W.make_projection(5, 600, 256, [96, 160], 4, 32, p_none=0.0,
                          token_to_slot=[i // 150 for i in range(600)])
    check_delta(p, run_delta(p, N.IMPL_AUTO, "eager"), "prefill, odd slices")


@pytest.mark.parametrize("name", ["qkv", "o", "gate_up", "down"])
def test_prefill_delta_is_stored_by_the_tile_kernel(name):
    p = W.prefill_projection(name, seed=2)
    check_delta(p, run_delta(p, N.IMPL_AUTO, "eager", pad=64), f"prefill {name}")


def test_prefill_delta_mixed_blocks_and_rows_without_adapter():
    """Runs of different slots inside one 128-row block, rows and whole blocks without adapter, ragged last block."""
    gen = torch.Generator().manual_seed(9)
    T, S = 1000, 6
    slots = torch.repeat_interleave(torch.randint(-1, S, (40,), generator=gen), 25)
    slots[256:512] = -1   # two whole row blocks without adapter
    p = W.make_projection(7, T, 512, [256, 128, 128], S, 64, ranks=[8, 16, 64, 64, 32, 16], token_to_slot=slots.tolist())
    check_delta(p, run_delta(p, N.IMPL_AUTO, "eager"), "mixed blocks")
    check_delta(p, run_delta(p, N.IMPL_SGMV, "eager"), "mixed blocks / SGMV")


@pytest.mark.parametrize("kind", ["qkv", "gate_up", "row"])
def test_layers_lora_first_order(kind):
    """LORA_FIRST: delta into the output buffer, then the base GEMM accumulates; same result as adding after the
    GEMM within the path's tolerance, rows without adapter bit-identical to the accumulate-into(-0.0) base GEMM."""
    torch.manual_seed(0)
    S, r, T = 6, 32, 48
    if kind == "qkv":
        layer = L.LoRAQKVParallelLinear(256, 64, 4, 2, max_loras=S, max_lora_rank=r)
    elif kind == "gate_up":
        layer = L.LoRAMergedColumnParallelLinear(256, [512, 512], max_loras=S, max_lora_rank=r)
    else:
        layer = L.LoRARowParallelLinear(512, 256, max_loras=S, max_lora_rank=r)
    layer = layer.to(DEV, torch.bfloat16)
    with torch.no_grad():
        layer.weight.normal_(0, 0.05)
        for name, prm in layer.named_parameters():
            if "lora_" in name:
                prm.normal_(0, 0.05)
    for s in range(S):
        layer._effective_lora_rank_values[s] = r
    layer.effective_lora_rank.fill_(r)
    x = torch.randn(T, layer.weight.size(1), device=DEV).to(torch.bfloat16)
    slots = torch.randint(-1, S, (T,), dtype=torch.int32)
    CTX.set_lora_context(CTX.build_lora_context_from_token_to_slot(slots.to(DEV)))
    with torch.inference_mode():
        after = layer(x)
        L.LORA_FIRST = True
        first = layer(x)
        L.LORA_FIRST = False
        base = torch.full_like(first, -0.0).addmm_(x, layer.weight.t())
    assert not torch.equal(after, base)
    assert_lora_close(first, after.float(), what=kind)
    none = slots < 0
    assert torch.equal(first[none].view(torch.int16), base[none].view(torch.int16))
    torch.testing.assert_close(first[none].float(), after[none].float(), atol=1e-2, rtol=1e-2)
