"""Phase timeline of the fused decode kernel inside a replayed CUDA graph (tuning aid).

    python -m nanovllm_voxcpm_b200.build --trace          # lib/libb200lora_trace.so (-DB200_TRACE)
    B200_LORA_LIB=nanovllm-voxcpm_b200/lib/libb200lora_trace.so python -m nanovllm_voxcpm_b200.timeline

For each projection of the decode configuration (256 rows, 32 adapters of rank 32) a graph of 16 launches over
16 distinct slab sets is replayed, so that the launches overlap as they do in a decoder step; the kernel of the
tuning build records SM-clock timestamps of its phases (first CTA of every bucket's cluster, last launch of the
replay). Printed: microseconds since the CTA started, median over the buckets, and the spread of the chain
that follows ``griddepcontrol.wait``. The tuning build is slower than the product build (each mark costs about
40 ns); the timeline shows proportions, ``bench.py`` gives the timed numbers.
"""

from __future__ import annotations

import ctypes

import torch

from . import _native as N
from . import batch_plan as BP
from . import lora as LORA
from . import workloads as W

LABELS = ["start", "bucket metadata", "barriers ready", "first ring issued (producer)", "wait returned",
          "first tile ready", "shrink done", "reduction barrier", "intermediate sent", "intermediate complete",
          "expand done", "end"]


def _graph_metadata(slots: torch.Tensor, n_slots: int, device) -> LORA.LoRAMetadata:
    bufs = BP.GraphLoRABuffers.make(slots.numel(), n_slots, device=device)
    bufs.load_plan(BP.build_lora_batch_plan_from_token_to_slot({}, slots.tolist()))
    ctx = bufs.context(slots.numel())
    return LORA.LoRAMetadata(ctx.token_to_slot, ctx.token_indices_sorted_by_slot, ctx.active_slot_ids,
                             ctx.num_tokens_per_slot, ctx.slot_start_offsets, False, ctx.num_active_loras)


def main(n_sets: int = 16, replays: int = 5, sm_mhz: float = 1965.0) -> None:
    lib = N.lib()
    if not hasattr(lib, "lora_b200_debug_trace"):
        raise SystemExit("this library was not built with -DB200_TRACE (python -m nanovllm_voxcpm_b200.build --trace, "
                         "then set B200_LORA_LIB to lib/libb200lora_trace.so)")
    lib.lora_b200_debug_trace.restype = ctypes.c_int32
    lib.lora_b200_debug_trace.argtypes = [ctypes.c_void_p, ctypes.c_int32]
    dev = torch.device("cuda", torch.cuda.current_device())
    slots = W.uniform_slots(torch.Generator().manual_seed(0), 256, 32, 0.1)
    meta = _graph_metadata(slots, 32, dev)
    gen = torch.Generator(device=dev).manual_seed(1)
    rn = lambda *s, std=0.02: (torch.randn(*s, generator=gen, device=dev) * std).to(torch.bfloat16)  # noqa: E731
    for name, (in_dim, outs) in W.DECODE_LAYER.items():
        sets = [dict(x=rn(256, in_dim, std=1.0), y=rn(256, sum(outs), std=1.0), a=[rn(32, 32, in_dim) for _ in outs],
                     b=[rn(32, o, 32) for o in outs]) for _ in range(n_sets)]
        cols = [sum(outs[:i]) for i in range(len(outs))]

        def step():
            for p in sets:
                LORA.launch_add(p["y"], p["x"], p["a"], p["b"], list(outs), cols, meta, 1.0, impl=N.IMPL_BGMV)

        stream = torch.cuda.Stream(dev)
        with torch.cuda.stream(stream):
            step()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step()
            for _ in range(3):
                graph.replay()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            for _ in range(replays):
                graph.replay()
            end.record(stream)
            end.synchronize()
        us = start.elapsed_time(end) * 1e3 / (replays * n_sets)
        buf = (ctypes.c_longlong * (33 * 32))()
        N.check(lib.lora_b200_debug_trace(buf, 33 * 32))
        marks = torch.tensor(list(buf), dtype=torch.float64).view(33, 32)[1:]  # bucket 0 of the graph buffers is the idle one
        rel = (marks - marks[:, :1]) / sm_mhz
        med = rel.median(0).values.tolist()
        chain = (marks[:, 11] - marks[:, 4]) / sm_mhz
        print(f"{name}: {us:.2f} us per launch (tuning build)")
        print("   " + ", ".join(f"{label} {v:.2f}" for label, v in zip(LABELS, med[:12])))
        print(f"   chain after the wait, over the 32 clusters: min {chain.min():.2f} / median {chain.median():.2f} / "
              f"max {chain.max():.2f} us")


if __name__ == "__main__":
    main()
