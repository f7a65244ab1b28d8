"""Decoder-step harness around the four LoRA linears (measurement only).

A MiniCPM-4 style pre-norm decoder with the structure of the reference's backbone
(``nanovllm_voxcpm/models/voxcpm2/model.py:109-334``: ``Cpm4Attention`` = qkv projection -> RoPE ->
paged attention -> o projection, ``Cpm4MLP`` = gate_up projection -> SiLU * up -> down projection,
``Cpm4DecoderLayer`` = RMSNorm + residual around both), random-init weights, input embeddings fed
directly. The four projections are this package's LoRA layers; attention and the paged KV cache go
through flash_attn (``flash_attn_varlen_func`` for prefill, ``flash_attn_with_kvcache`` with a block
table for decode), as in the reference (``layers/attention.py:10-79``). The steps in between
(residual add + RMSNorm, RoPE + cache store, SiLU * up) run as plain torch ops, or, with
``Decoder.fused_glue = True``, as the single-launch kernels of ``glue.py``.

It exists to time a whole step with the multi-LoRA kernels in their real surroundings (one prefill
step over all prompts, then decode steps replayed from a CUDA graph) and to compare it with the same
step without adapters.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import glue as G
from . import layers as L
from . import lora as LORA
from .batch_plan import GraphLoRABuffers, build_lora_batch_plan_from_token_to_slot, build_lora_context_from_batch_plan
from .context import LoRAContext, build_mixed_lora_context, reset_lora_context, set_lora_context


@dataclass
class DecoderConfig:
    hidden_size: int = 1024
    num_heads: int = 16
    num_kv_heads: int = 2
    head_dim: int = 64
    intermediate_size: int = 4096
    num_layers: int = 24
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position: int = 4096
    max_loras: int = 128
    max_lora_rank: int = 32
    kv_block_size: int = 256
    #: how the row-parallel layers (o, down) handle their LoRA delta under tensor parallelism
    #: (``layers.LoRARowParallelLinear``): "partial_y" (the reference's), "allreduce_tmp", "peer_exchange"
    lora_tp_mode: str = "partial_y"


@dataclass
class AttentionStep:
    """Per-step attention inputs (the reference keeps them in a global context, ``utils/context.py:38-74``)."""

    is_prefill: bool
    slot_mapping: torch.Tensor          # int64 [T]  flat cache position of every new token
    cu_seqlens: torch.Tensor | None = None     # int32 [B+1]  (prefill)
    max_seqlen: int = 0
    context_lens: torch.Tensor | None = None   # int32 [B]    (decode, new token included)
    block_tables: torch.Tensor | None = None   # int32 [B, blocks per request]
    #: mixed step (``is_prefill`` True and ``n_decode`` > 0): rows ``[0, n_decode)`` are single-token decode rows
    #: (``context_lens`` / ``block_tables`` describe them), the rest is a prefill chunk (``cu_seqlens``)
    n_decode: int = 0


def _rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    # x [T, heads, head_dim], cos / sin [T, 1, head_dim / 2]; rotate-half form
    x1, x2 = x.float().chunk(2, dim=-1)
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).to(x.dtype)


class DecoderAttention(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg
        tp = L._get_world_size()  # heads are split over the tensor-parallel ranks, as the layers split their weights
        self.heads, self.kv_heads = L.divide(cfg.num_heads, tp), L.divide(cfg.num_kv_heads, tp)
        self.q_size = self.heads * cfg.head_dim
        self.kv_size = self.kv_heads * cfg.head_dim
        self.qkv_proj = L.LoRAQKVParallelLinear(cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.num_kv_heads,
                                                max_loras=cfg.max_loras, max_lora_rank=cfg.max_lora_rank)
        self.o_proj = L.LoRARowParallelLinear(cfg.num_heads * cfg.head_dim, cfg.hidden_size, max_loras=cfg.max_loras,
                                              max_lora_rank=cfg.max_lora_rank, lora_tp_mode=cfg.lora_tp_mode)
        self.k_cache = self.v_cache = None  # [blocks, block_size, kv_heads, head_dim], set by the harness

    def forward(self, positions, hidden, step: AttentionStep, cos_sin) -> torch.Tensor:
        cfg = self.cfg
        qkv = self.qkv_proj(hidden)
        q, k, v = qkv.split([self.q_size, self.kv_size, self.kv_size], dim=-1)
        cos, sin = cos_sin
        q = _rope(q.view(-1, self.heads, cfg.head_dim), cos, sin)
        k = _rope(k.view(-1, self.kv_heads, cfg.head_dim), cos, sin)
        v = v.reshape(-1, self.kv_heads, cfg.head_dim)
        flat_k = self.k_cache.view(-1, self.kv_heads, cfg.head_dim)
        flat_v = self.v_cache.view(-1, self.kv_heads, cfg.head_dim)
        flat_k.index_copy_(0, step.slot_mapping, k)
        flat_v.index_copy_(0, step.slot_mapping, v)
        return self.o_proj(self._attend(q, k, v, step).reshape(-1, self.q_size))

    def _attend(self, q, k, v, step: AttentionStep) -> torch.Tensor:
        """flash_attn over the paged cache (decode rows) and / or the packed prompts (prefill rows)."""
        from flash_attn import flash_attn_varlen_func, flash_attn_with_kvcache

        scale = self.cfg.head_dim ** -0.5
        nd = step.n_decode if step.is_prefill else q.size(0)
        outs = []
        if nd:
            outs.append(flash_attn_with_kvcache(q[:nd].unsqueeze(1), self.k_cache, self.v_cache, cache_seqlens=step.context_lens,
                                                block_table=step.block_tables, softmax_scale=scale, causal=True).squeeze(1))
        if step.is_prefill:
            outs.append(flash_attn_varlen_func(q[nd:], k[nd:], v[nd:], step.cu_seqlens, step.cu_seqlens, step.max_seqlen,
                                               step.max_seqlen, softmax_scale=scale, causal=True))
        return outs[0] if len(outs) == 1 else torch.cat(outs, dim=0)

    def forward_fused(self, positions, normed, step: AttentionStep, cos, sin, slot_mapping_i32) -> torch.Tensor:
        """Same as ``forward`` with RoPE and the cache store as one in-place kernel over the packed qkv rows."""
        cfg = self.cfg
        q, k, v = G.rope_kv_store(self.qkv_proj(normed), self.heads, self.kv_heads, cfg.head_dim, positions=positions,
                                  cos=cos, sin=sin, k_cache=self.k_cache, v_cache=self.v_cache, slot_mapping=slot_mapping_i32)
        return self.o_proj(self._attend(q, k, v, step).reshape(-1, self.q_size))


class DecoderMLP(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.gate_up_proj = L.LoRAMergedColumnParallelLinear(cfg.hidden_size, [cfg.intermediate_size] * 2,
                                                             max_loras=cfg.max_loras, max_lora_rank=cfg.max_lora_rank)
        self.down_proj = L.LoRARowParallelLinear(cfg.intermediate_size, cfg.hidden_size, max_loras=cfg.max_loras,
                                                 max_lora_rank=cfg.max_lora_rank, lora_tp_mode=cfg.lora_tp_mode)

    def forward(self, x):
        gate, up = self.gate_up_proj(x).chunk(2, dim=-1)
        return self.down_proj(F.silu(gate) * up)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg
        self.self_attn = DecoderAttention(cfg)
        self.mlp = DecoderMLP(cfg)
        self.input_layernorm = nn.Parameter(torch.ones(cfg.hidden_size))
        self.post_attention_layernorm = nn.Parameter(torch.ones(cfg.hidden_size))

    def forward(self, positions, hidden, step, cos_sin):
        eps = self.cfg.rms_norm_eps
        hidden = hidden + self.self_attn(positions, _rms_norm(hidden, self.input_layernorm, eps), step, cos_sin)
        return hidden + self.mlp(_rms_norm(hidden, self.post_attention_layernorm, eps))


class Decoder(nn.Module):
    """``num_layers`` decoder layers + final norm over input embeddings ``[T, hidden]``."""

    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg
        self.layers = nn.ModuleList([DecoderLayer(cfg) for _ in range(cfg.num_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size))
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float32) / cfg.head_dim))
        freqs = torch.outer(torch.arange(cfg.max_position, dtype=torch.float32), inv)
        self.register_buffer("cos", freqs.cos(), persistent=False)
        self.register_buffer("sin", freqs.sin(), persistent=False)

    #: True: the steps between the projections run as this package's single-launch kernels (``glue.py``):
    #: residual add + RMSNorm, RoPE + cache store, SiLU * up; False: plain torch ops
    fused_glue = False

    def _forward_fused(self, embeds, positions, step: AttentionStep):
        eps = self.cfg.rms_norm_eps
        slot_i32 = step.slot_mapping.to(torch.int32)
        hidden = embeds
        normed, _ = G.add_rms_norm(hidden, None, self.layers[0].input_layernorm, eps)
        for i, layer in enumerate(self.layers):
            attn = layer.self_attn.forward_fused(positions, normed, step, self.cos, self.sin, slot_i32)
            normed, hidden = G.add_rms_norm(attn, hidden, layer.post_attention_layernorm, eps)
            down = layer.mlp.down_proj(G.silu_and_mul(layer.mlp.gate_up_proj(normed)))
            following = self.layers[i + 1].input_layernorm if i + 1 < len(self.layers) else self.norm
            normed, hidden = G.add_rms_norm(down, hidden, following, eps)
        return normed

    def forward(self, embeds, positions, step: AttentionStep):
        if self.fused_glue:
            return self._forward_fused(embeds, positions, step)
        cos_sin = (self.cos[positions].unsqueeze(1), self.sin[positions].unsqueeze(1))
        hidden = embeds
        for layer in self.layers:
            hidden = layer(positions, hidden, step, cos_sin)
        return _rms_norm(hidden, self.norm, self.cfg.rms_norm_eps)

    # ------------------------------------------------------------------ set-up helpers
    def init_random_(self, seed: int = 0, std: float = 0.02) -> None:
        gen = torch.Generator(device=self.norm.device).manual_seed(seed)
        with torch.no_grad():
            for mod in L.iter_lora_modules(self):
                mod.weight.normal_(0.0, std, generator=gen)

    def fill_adapter_slots_(self, n_slots: int, rank: int, seed: int = 1, std: float = 0.02) -> None:
        """Random rank-``rank`` adapters in slots ``0..n_slots-1`` of every LoRA module: slab rows /
        columns ``[:rank]`` random, the rest zero, rank buffers set (what ``set_slot_lora`` leaves
        behind, written slab-wide instead of slot by slot)."""
        gen = torch.Generator(device=self.norm.device).manual_seed(seed)
        with torch.no_grad():
            for mod in L.iter_lora_modules(self):
                for slab in mod._a_slices():
                    slab.zero_()
                    slab[:n_slots, :rank].normal_(0.0, std, generator=gen)
                for slab in mod._b_slices():
                    slab.zero_()
                    slab[:n_slots, :, :rank].normal_(0.0, std, generator=gen)
                for s in range(n_slots):
                    mod._effective_lora_rank_values[s] = rank
                    mod._lora_scaling_values[s] = mod._lora_base_scaling_values[s] = 1.0
                mod.effective_lora_rank[:n_slots] = rank
                mod.lora_scaling[:n_slots] = 1.0
                mod.lora_base_scaling[:n_slots] = 1.0

    def attach_tp_exchange(self, exchange) -> None:
        """One ``TpExchange`` shared by the row-parallel layers (``lora_tp_mode="peer_exchange"``)."""
        for layer in self.layers:
            layer.self_attn.o_proj.tp_exchange = exchange
            layer.mlp.down_proj.tp_exchange = exchange

    def load_full_random_(self, n_slots: int, rank: int, seed: int = 0, std: float = 0.02) -> None:
        """Full (unsharded) random base weights and adapters drawn from one seeded generator, the same on every
        rank, loaded through the layers' own shard loaders: a tensor-parallel model and a single-GPU model built
        with the same seed then compute the same function. Meant for small parity cases (every rank materialises
        the full tensors)."""
        dev = self.norm.device
        gen = torch.Generator(device=dev).manual_seed(seed)
        dt = self.layers[0].self_attn.qkv_proj.weight.dtype
        rn = lambda *shape: (torch.randn(*shape, generator=gen, device=dev) * std).to(dt)  # noqa: E731
        cfg = self.cfg
        hq, hkv = cfg.num_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
        with torch.no_grad():
            for layer in self.layers:
                qkv, o, gu, down = layer.self_attn.qkv_proj, layer.self_attn.o_proj, layer.mlp.gate_up_proj, layer.mlp.down_proj
                for shard, rows in (("q", hq), ("k", hkv), ("v", hkv)):
                    qkv.load_base_shard(rn(rows, cfg.hidden_size), shard)
                o.load_base_shard(rn(cfg.hidden_size, hq))
                for i in range(2):
                    gu.load_base_shard(rn(cfg.intermediate_size, cfg.hidden_size), i)
                down.load_base_shard(rn(cfg.hidden_size, cfg.intermediate_size))
                tp, r = qkv.tp_size, qkv.tp_rank
                for slot in range(n_slots):
                    a = rn(3, rank, cfg.hidden_size)
                    b = [rn(rows, rank).chunk(tp, 0)[r] for rows in (hq, hkv, hkv)]
                    qkv.set_slot_lora(slot, a, b, rank, 1.0)
                    a = rn(2, rank, cfg.hidden_size)
                    b = [rn(cfg.intermediate_size, rank).chunk(tp, 0)[r] for _ in range(2)]
                    gu.set_slot_lora(slot, a, b, rank, 1.0)
                    for mod, width in ((o, hq), (down, cfg.intermediate_size)):
                        a, b = rn(rank, width).chunk(tp, 1)[r], rn(cfg.hidden_size, rank)
                        if mod.lora_tp_mode != "partial_y":
                            b = b.chunk(tp, 0)[r]
                        mod.set_slot_lora(slot, a.contiguous(), b.contiguous(), rank, 1.0)

    def allocate_kv_cache(self, num_blocks: int) -> None:
        cfg = self.cfg
        dev, dt = self.norm.device, self.layers[0].self_attn.qkv_proj.weight.dtype
        kv_heads = self.layers[0].self_attn.kv_heads
        for layer in self.layers:
            layer.self_attn.k_cache = torch.zeros(num_blocks, cfg.kv_block_size, kv_heads, cfg.head_dim, device=dev, dtype=dt)
            layer.self_attn.v_cache = torch.zeros_like(layer.self_attn.k_cache)


# ---------------------------------------------------------------------- the serving loop of the harness
@dataclass
class BackboneWorkload:
    prompt_lens: list[int]
    adapter_of_request: list[int]      # slot id per request (-1 = none)
    decode_steps: int


def zipf_adapters(n_requests: int, n_adapters: int, s: float = 1.1, seed: int = 0) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    w = 1.0 / torch.arange(1, n_adapters + 1, dtype=torch.float64) ** s
    return torch.multinomial(w / w.sum(), n_requests, replacement=True, generator=gen).tolist()


class BackboneRunner:
    """Prefill of all prompts (in chunks of whole requests) and graph-replayed decode steps."""

    def __init__(self, model: Decoder, work: BackboneWorkload, use_lora: bool = True, max_prefill_tokens: int = 8192):
        self.model, self.work, self.use_lora = model, work, use_lora
        cfg = model.cfg
        self.dev = model.norm.device
        self.B = len(work.prompt_lens)
        self.max_prefill_tokens = max_prefill_tokens
        per_req = -(-(max(work.prompt_lens) + work.decode_steps + 1) // cfg.kv_block_size)
        model.allocate_kv_cache(self.B * per_req)
        self.block_tables = torch.arange(self.B * per_req, dtype=torch.int32, device=self.dev).view(self.B, per_req)
        self.slots = torch.tensor(work.adapter_of_request, dtype=torch.int32)
        self.dtype = model.layers[0].self_attn.qkv_proj.weight.dtype

    def _cache_positions(self, req: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        bs = self.model.cfg.kv_block_size
        blk = self.block_tables[req.long(), (pos // bs).long()].long()
        return blk * bs + (pos % bs).long()

    @torch.inference_mode()
    def prefill(self, embeds_of: dict[int, torch.Tensor] | None = None) -> tuple[int, float]:
        """Runs every prompt through the model; returns (tokens, milliseconds on the device)."""
        chunks, cur, cur_tokens = [], [], 0
        for i, n in enumerate(self.work.prompt_lens):
            if cur and cur_tokens + n > self.max_prefill_tokens:
                chunks.append(cur)
                cur, cur_tokens = [], 0
            cur.append(i)
            cur_tokens += n
        if cur:
            chunks.append(cur)
        gen = torch.Generator(device=self.dev).manual_seed(7)
        steps = []
        for reqs in chunks:
            lens = [self.work.prompt_lens[i] for i in reqs]
            T = sum(lens)
            req = torch.repeat_interleave(torch.tensor(reqs), torch.tensor(lens)).to(self.dev)
            pos = torch.cat([torch.arange(n) for n in lens]).to(self.dev)
            cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=self.dev)
            embeds = torch.randn(T, self.model.cfg.hidden_size, device=self.dev, generator=gen).to(self.dtype)
            step = AttentionStep(True, self._cache_positions(req, pos), cu_seqlens=cu, max_seqlen=max(lens))
            tts = torch.repeat_interleave(self.slots[torch.tensor(reqs)], torch.tensor(lens))
            ctx = None
            if self.use_lora:
                ctx = build_lora_context_from_batch_plan(
                    build_lora_batch_plan_from_token_to_slot({}, tts.tolist()), device=self.dev)
            steps.append((embeds, pos, step, ctx))
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for embeds, pos, step, ctx in steps:
            set_lora_context(ctx) if ctx is not None else reset_lora_context()
            self.last_output = self.model(embeds, pos, step)
        end.record()
        end.synchronize()
        reset_lora_context()
        return sum(self.work.prompt_lens), start.elapsed_time(end)

    @torch.inference_mode()
    def decode(self, steps: int | None = None, use_graph: bool = True) -> tuple[int, float, str]:
        """``steps`` decode steps of one token per request; returns (tokens, milliseconds, launch mode)."""
        steps = steps or self.work.decode_steps
        cfg = self.model.cfg
        B = self.B
        req = torch.arange(B, device=self.dev)
        pos = torch.tensor(self.work.prompt_lens, device=self.dev)          # position of the next token
        gen = torch.Generator(device=self.dev).manual_seed(11)
        embeds = torch.randn(B, cfg.hidden_size, device=self.dev, generator=gen).to(self.dtype)
        slot_mapping = self._cache_positions(req, pos)
        context_lens = (pos + 1).to(torch.int32)
        step = AttentionStep(False, slot_mapping, context_lens=context_lens, block_tables=self.block_tables)
        if self.use_lora:
            bufs = GraphLoRABuffers.make(B, cfg.max_loras, device=self.dev)
            bufs.load_token_to_slot_on_device(self.slots.to(self.dev))
            set_lora_context(bufs.context(B))
        else:
            reset_lora_context()
        out = torch.empty_like(embeds)

        def one_step():
            out.copy_(self.model(embeds, pos, step))

        def advance():  # device-side bookkeeping between steps (no host sync)
            embeds.copy_(out)
            pos.add_(1)
            context_lens.add_(1)
            slot_mapping.copy_(self._cache_positions(req, pos))

        stream = torch.cuda.Stream(self.dev)
        mode = "eager"
        with torch.cuda.stream(stream):
            for _ in range(3):
                one_step()
            stream.synchronize()
            run = one_step
            if use_graph:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    one_step()
                run, mode = graph.replay, "cuda_graph"
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            stream.synchronize()
            start.record(stream)
            for _ in range(steps):
                run()
                advance()
            end.record(stream)
            end.synchronize()
        reset_lora_context()
        self.last_output = out
        return B * steps, start.elapsed_time(end), mode


@torch.inference_mode()
def time_mixed_step(model: Decoder, n_decode: int, prefill_lens: list[int], slots_decode: list[int], slots_prefill: list[int],
                    context_len: int = 200, iters: int = 5, warmup: int = 2, use_lora: bool = True, seed: int = 3):
    """One continuous-batching step that holds ``n_decode`` single-token decode rows (requests with ``context_len``
    tokens in the paged cache) AND a prefill chunk of whole prompts (``prefill_lens``), as a scheduler that mixes
    the two kinds builds it: rows ``[0, n_decode)`` decode, then the prompts packed. Attention runs per kind
    (paged decode / varlen prefill); every LoRA layer issues one multi-LoRA call per kind
    (``LoRAContext.parts``). Returns (tokens per step, milliseconds per step on the device, last output)."""
    cfg, dev = model.cfg, model.norm.device
    dtype = model.layers[0].self_attn.qkv_proj.weight.dtype
    bs = cfg.kv_block_size
    per_decode = -(-(context_len + 1) // bs)
    blocks_prefill = [-(-n // bs) for n in prefill_lens]
    model.allocate_kv_cache(n_decode * per_decode + sum(blocks_prefill))
    block_tables = torch.arange(n_decode * per_decode, dtype=torch.int32, device=dev).view(n_decode, per_decode)
    T_pre = sum(prefill_lens)
    # cache position of every new token
    dec_pos = block_tables[:, context_len // bs].long() * bs + context_len % bs
    first = n_decode * per_decode
    pre_pos, positions = [], [torch.full((n_decode,), context_len, dtype=torch.int64)]
    for n, nb in zip(prefill_lens, blocks_prefill):
        pre_pos.append(first * bs + torch.arange(n))
        positions.append(torch.arange(n))
        first += nb
    slot_mapping = torch.cat([dec_pos.cpu(), *pre_pos]).to(dev)
    positions = torch.cat(positions).to(dev)
    cu = torch.tensor([0] + list(torch.tensor(prefill_lens).cumsum(0)), dtype=torch.int32, device=dev)
    step = AttentionStep(True, slot_mapping, cu_seqlens=cu, max_seqlen=max(prefill_lens),
                         context_lens=torch.full((n_decode,), context_len + 1, dtype=torch.int32, device=dev),
                         block_tables=block_tables, n_decode=n_decode)
    gen = torch.Generator(device=dev).manual_seed(seed)
    embeds = torch.randn(n_decode + T_pre, cfg.hidden_size, device=dev, generator=gen).to(dtype)
    tts = torch.cat([torch.tensor(slots_decode, dtype=torch.int32),
                     torch.repeat_interleave(torch.tensor(slots_prefill, dtype=torch.int32), torch.tensor(prefill_lens))])
    ctx = build_mixed_lora_context(tts.to(dev), [n_decode]) if use_lora else None
    out = None
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(warmup + iters):
        if i == warmup:
            torch.cuda.synchronize()
            start.record()
        set_lora_context(ctx) if ctx is not None else reset_lora_context()
        out = model(embeds, positions, step)
    end.record()
    end.synchronize()
    reset_lora_context()
    return n_decode + T_pre, start.elapsed_time(end) / iters, out
