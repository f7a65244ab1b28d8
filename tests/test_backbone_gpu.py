"""The decoder-step harness around the LoRA linears: the kernels inside a real layer stack
(prefill through the tensor-core path, decode through the fused kernel, eager and graph replay)
against the same stack with the CPU-oracle formula as LoRA backend."""

import pytest
import torch

from helpers import OracleBackend
from nanovllm_voxcpm_b200 import _native as N
from nanovllm_voxcpm_b200 import backbone as BB
from nanovllm_voxcpm_b200 import context as CTX
from nanovllm_voxcpm_b200 import lora as LORA

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _clean():
    LORA.set_backend_for_testing(None)
    CTX.reset_lora_context()
    yield
    LORA.set_backend_for_testing(None)
    CTX.reset_lora_context()
    assert N.device_status() == 0


def _model_and_work():
    pytest.importorskip("flash_attn")
    cfg = BB.DecoderConfig(hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=512,
                           num_layers=2, max_loras=8, max_lora_rank=32, max_position=1024)
    with torch.device("cuda"):
        model = BB.Decoder(cfg).to(torch.bfloat16)
    model.init_random_(0, std=0.05)
    model.fill_adapter_slots_(8, 32, seed=1, std=0.05)
    # 600 prompt rows: the prefill batch takes the tcgen05 kernels (>= 512 rows), with a request without adapter
    work = BB.BackboneWorkload([200, 17, 264, 5, 114], [0, 3, -1, 3, 7], decode_steps=3)
    return model, work


def test_backbone_prefill_and_decode_match_the_oracle_backend():
    model, work = _model_and_work()
    mine = BB.BackboneRunner(model, work, use_lora=True)
    mine.prefill()
    out_prefill = mine.last_output.float().cpu()
    mine.decode(3, use_graph=True)
    out_graph = mine.last_output.float().cpu()

    eager = BB.BackboneRunner(model, work, use_lora=True)
    eager.prefill()
    eager.decode(3, use_graph=False)
    assert torch.equal(out_graph, eager.last_output.float().cpu()), "graph replay and eager launches differ"

    base = BB.BackboneRunner(model, work, use_lora=False)
    base.prefill()
    out_base = base.last_output.float().cpu()
    assert not torch.allclose(out_prefill, out_base, atol=1e-3), "adapters changed nothing"

    LORA.set_backend_for_testing(OracleBackend())
    ref = BB.BackboneRunner(model, work, use_lora=True)
    ref.prefill()
    ref_prefill = ref.last_output.float().cpu()
    ref.decode(3, use_graph=False)
    ref_decode = ref.last_output.float().cpu()
    # two bf16 layers around the op: tolerance of the stack, not of the kernel
    torch.testing.assert_close(out_prefill, ref_prefill, atol=6e-2, rtol=6e-2)
    torch.testing.assert_close(out_graph, ref_decode, atol=6e-2, rtol=6e-2)
    # the request without adapter sees exactly the base model in prefill (rows 217..480 of the single chunk)
    assert torch.equal(out_prefill[217:481], out_base[217:481])


def test_mixed_step_splits_decode_rows_and_prefill_chunk():
    """A step that holds single-token decode rows AND a prefill chunk: every LoRA layer issues one call per row
    range (``LoRAContext.parts``), attention runs per kind. Against the same step with the oracle formula as the
    LoRA backend (which sees each range under its own context too), and against the step without adapters on the
    rows that have none."""
    model, _ = _model_and_work()
    n_dec, lens = 24, [300, 230, 70]  # 600 prefill rows: tensor-core kernels; 24 decode rows: fused decode kernel
    gen = torch.Generator().manual_seed(4)
    dec = torch.randint(-1, 8, (n_dec,), generator=gen).tolist()
    pre = [2, -1, 5]
    for fused in (False, True):
        model.fused_glue = fused
        try:
            tokens, _, out = BB.time_mixed_step(model, n_dec, lens, dec, pre, context_len=40, iters=1, warmup=1)
            _, _, base = BB.time_mixed_step(model, n_dec, lens, dec, pre, context_len=40, iters=1, warmup=1, use_lora=False)
            LORA.set_backend_for_testing(OracleBackend())
            _, _, ref = BB.time_mixed_step(model, n_dec, lens, dec, pre, context_len=40, iters=1, warmup=1)
        finally:
            LORA.set_backend_for_testing(None)
            model.fused_glue = False
        assert tokens == n_dec + sum(lens)
        torch.testing.assert_close(out.float(), ref.float(), atol=6e-2, rtol=6e-2)
        rows = torch.tensor([i for i, s in enumerate(dec) if s < 0] + list(range(n_dec + 300, n_dec + 530)), device="cuda")
        assert torch.equal(out[rows], base[rows]), "rows without adapter differ from the model without adapters"
        assert not torch.allclose(out.float(), base.float(), atol=1e-3)


def test_fused_glue_step_matches_the_torch_glue_step():
    """The same decoder with residual add + RMSNorm, RoPE + cache store and SiLU * up as single launches: outputs
    within the rounding of a two-layer bf16 stack, KV caches equal, graph replay equal to eager launches."""
    model, work = _model_and_work()
    plain = BB.BackboneRunner(model, work, use_lora=True)
    plain.prefill()
    plain_prefill = plain.last_output.float().cpu()
    plain_k = model.layers[0].self_attn.k_cache.clone()
    plain.decode(3, use_graph=False)
    plain_decode = plain.last_output.float().cpu()
    try:
        model.fused_glue = True
        fused = BB.BackboneRunner(model, work, use_lora=True)  # allocates fresh caches
        fused.prefill()
        fused_prefill = fused.last_output.float().cpu()
        # layer 0's cache holds the rotated k of the first projection: same inputs up to the norm's last place
        torch.testing.assert_close(model.layers[0].self_attn.k_cache.float(), plain_k.float(), atol=2e-2, rtol=2e-2)
        fused.decode(3, use_graph=True)
        fused_graph = fused.last_output.float().cpu()
        eager = BB.BackboneRunner(model, work, use_lora=True)
        eager.prefill()
        eager.decode(3, use_graph=False)
        assert torch.equal(fused_graph, eager.last_output.float().cpu())
    finally:
        model.fused_glue = False
    torch.testing.assert_close(fused_prefill, plain_prefill, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(fused_graph, plain_decode, atol=3e-2, rtol=3e-2)


def test_lora_first_order_in_the_decode_graph():
    """Decode steps with the delta written before the base GEMM (layers.LORA_FIRST): graph replay equals eager
    launches bit for bit, and the result stays within the stack's tolerance of the add-after-GEMM order."""
    from nanovllm_voxcpm_b200 import layers as L

    model, work = _model_and_work()
    outs = {}
    try:
        model.fused_glue = True
        for order in ("after", "first", "first_eager"):
            L.LORA_FIRST = order != "after"
            run = BB.BackboneRunner(model, work, use_lora=True)
            run.prefill()
            run.decode(3, use_graph=order != "first_eager")
            outs[order] = run.last_output.float().cpu()
    finally:
        model.fused_glue = False
        L.LORA_FIRST = False
    assert torch.equal(outs["first"], outs["first_eager"])
    torch.testing.assert_close(outs["first"], outs["after"], atol=3e-2, rtol=3e-2)
