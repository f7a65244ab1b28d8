"""Benchmark of the multi-LoRA linear hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload (N=1 headline): the decode BGMV configuration - 256 sequences x 1 token through
the LoRA ops of a MiniCPM-style layer (hidden 1024, qkv out 1280, intermediate 4096; qkv /
o / gate_up / down, 7 projections), 32 adapters of rank 32 in bf16, slots uniform with 10 %
of rows without adapter.  One STEP = the four multi-LoRA launches of each of 24 layers
(96 launches) over 24 distinct slab sets (1.07 GB), so the weights of a launch are never
in L2 from the previous step (126 MB L2): inputs larger than L2 is the cache-defeat method.

  value      GB/s of ALGORITHMIC bytes (each active slot's A and B once, x rows, y read +
             write for rows with an adapter) with everything resident in HBM; the step is
             replayed as one CUDA graph and timed with CUDA events.
  e2e        the same metric through the public backend call (`B200LoRABackend.add_lora`)
             with host buffers: every layer's x and y come from pinned host memory (one packed
             copy per layer) and its y goes back to the host, all inside the timed region;
             copies and launches are pipelined over three streams.
  roofline   HBM roofline of the dominant kernel (bgmv_fused_kernel): algorithmic bytes per
             launch / average launch duration, against the measured copy bandwidth.
  cpu_baseline / --impl reference
             the reference's pure-PyTorch per-slot LoRA formula (the CPU oracle) on the
             host cores, on a bounded sample of the same workload (one layer per step).

With N > 1 (torchrun) every rank runs the same workload on its own GPU (request-level
replicas, no data-path collective): weak scaling, value = sum over ranks / max time.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "multi-LoRA linear GB/s (decode BGMV, algorithmic bytes)"
N_LAYERS = 24
T_DECODE, N_SLOTS, RANK, P_NONE = 256, 32, 32, 0.1
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference-gpu"],
                    help="b200 = this library; reference = the CPU restatement of the reference's op on the host cores; "
                         "reference-gpu = the unmodified reference's own GPU backend (its Triton kernels) from "
                         "baseline/_ref on the same workload, where that install and triton are usable")
    ap.add_argument("--layers", type=int, default=N_LAYERS)
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--glue", default="fused", choices=["fused", "torch"],
                    help="backbone workload: the steps between the projections as this library's single-launch kernels "
                         "(residual add + RMSNorm, RoPE + cache store, SiLU * up) or as plain torch ops")
    ap.add_argument("--lora-order", default="first", choices=["first", "after"],
                    help="backbone workload, decode steps: multi-LoRA delta written before the base GEMM, which then "
                         "accumulates into it (first), or added after the GEMM as the reference does (after)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--parallelism", default="tp", choices=["tp", "replicas"],
                    help="--workload backbone5 under torchrun: one tensor-parallel group, or one replica per GPU")
    ap.add_argument("--slab-gb", type=float, default=80.0, help="--workload backbone5: HBM budget of the adapter slabs per GPU")
    ap.add_argument("--no-base", action="store_true", help="--workload backbone5: skip the run without adapters")
    ap.add_argument("--extras-limit", type=float, default=420.0,
                    help="seconds after which the additional blocks of the line are cut short and the line is printed without them")
    ap.add_argument("--no-extras", action="store_true",
                    help="decode workload: only the headline measurement (no secondary / reference_gpu / backbone / tp blocks)")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "linear", "backbone", "backbone5", "tp", "admission", "glue"],
                    help="decode = the headline decode BGMV layer; prefill = prefill SGMV add (tcgen05 kernels) of one "
                         "layer; linear = base GEMM + LoRA in one tensor-core kernel for the same layer; backbone = whole "
                         "decoder steps (prefill + graph-replayed decode) around the LoRA linears")
    ap.add_argument("--only", default=None, choices=["qkv", "o", "gate_up", "down"],
                    help="tuning: time one projection of every layer instead of all four")
    ap.add_argument("--option", action="append", default=[], metavar="KEY=VALUE",
                    help="tuning: lora_b200_set_option before the run (cluster, pdl, ring_kb, ksplit)")
    return ap.parse_args()


def apply_options(args):
    """--option key=value -> lora_b200_set_option (tuning runs and profiler captures)."""
    from nanovllm_voxcpm_b200 import _native as N

    keys = {"cluster": N.OPT_CLUSTER, "pdl": N.OPT_PDL, "ring_kb": N.OPT_RING_KB,
            "ksplit": N.OPT_KSPLIT}
    for item in args.option:
        key, _, value = item.partition("=")
        N.set_option(keys[key], int(value))


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def config_dict(layers):
    return {
        "workload": "decode_bgmv: 256 seq x 1 token, hidden 1024, qkv 1280, inter 4096, 7 projections, "
                    "32 adapters rank 32 bf16, 10% rows without adapter",
        "layers_per_step": layers,
        "launches_per_step": 4 * layers,
        "cache_defeat": "inputs larger than L2 (distinct slab set per layer, %.2f GB per step)" % (layers * 44.56e6 / 1e9),
        "metadata": "cuda-graph buffers (max_loras+1 buckets)",
        "parallelism": "replicas",
    }


# ------------------------------------------------------------------ CPU baseline
def cpu_layer_inputs(seed=0):
    from nanovllm_voxcpm_b200 import workloads as W

    projs = [W.decode_projection(name, seed=seed + i, T=T_DECODE, S=N_SLOTS, r=RANK, p_none=P_NONE)
             for i, name in enumerate(W.DECODE_LAYER)]
    slots = projs[0].token_to_slot
    for p in projs:
        p.token_to_slot = slots
    return projs


def time_cpu_oracle(steps, warmup, budget_s=None, config="decode"):
    """Reference formula on the host cores. One step = one layer (4 projections) of the decode configuration, the
    single T = 64 linear of the CPU reference configuration (`config="reference_op"`), or one layer of the prefill
    configuration (`config="prefill"`)."""
    from nanovllm_voxcpm_b200 import workloads as W
    from oracle import lora_oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    if config == "reference_op":
        projs = [W.config1(seed=0)]
    elif config == "prefill":
        projs = [W.prefill_projection(name, seed=0) for name in W.PREFILL_LAYER]
    else:
        projs = cpu_layer_inputs()
    # fp32 copies so the timed part is the formula, not dtype conversion
    prepared = [(p.y.float(), p.x.float(), [a.float() for a in p.a_slabs], [b.float() for b in p.b_slabs],
                 p.token_to_slot, p.col_offsets) for p in projs]
    nbytes = sum(W.algorithmic_bytes(p) for p in projs)

    def step():
        for y, x, a, b, slots, cols in prepared:
            O.add_lora(y, x, a, b, slots, 1.0, cols)

    for _ in range(warmup):
        step()
    times = []
    t_begin = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
        if budget_s is not None and time.perf_counter() - t_begin > budget_s:
            break
    med = statistics.median(times)
    return dict(gbs=nbytes / med / 1e9, ms=med * 1e3, iters=len(times), bytes=nbytes, cores=torch.get_num_threads())


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = time_cpu_oracle(args.steps, args.warmup)
    sample = "one layer (4 multi-LoRA projections, 58 MB algorithmic) per step, fp32, torch CPU, per-slot formula"
    line = {
        "impl": "reference", "metric": METRIC, "value": r["gbs"], "unit": "GB/s", "n_gpus": args.gpus,
        "steps": r["iters"], "warmup": args.warmup, "ms_per_step": r["ms"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_dict(args.layers),
        "cpu_baseline": {"value": r["gbs"], "unit": "GB/s", "cores": r["cores"], "kind": "port", "sample": sample},
        "e2e": {"value": r["gbs"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------- GPU arm
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for row in open(self.path):
                f = [c.strip() for c in row.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        return out


def bind_to_gpu_cpus(index):
    """Pins this process to the CPUs that NVML reports as closest to GPU `index` (its NUMA node), so that pinned
    host buffers and the copy engines' traffic stay on that node. A setting of this process only. Returns a
    short description for the JSON line."""
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return "no CPU of the GPU's node is available to this process"
        os.sched_setaffinity(0, cpus)
        return f"{len(cpus)} CPUs of the GPU's NUMA node"
    except Exception as exc:  # NVML missing or not permitted: run unbound
        return f"unbound ({type(exc).__name__})"


def build_gpu_workload(device, layers):
    """Per layer and projection: device-resident x, y, slabs (distinct per layer)."""
    from nanovllm_voxcpm_b200 import workloads as W

    gen = torch.Generator(device=device).manual_seed(1234)
    cpu_gen = torch.Generator().manual_seed(0)
    slots = W.uniform_slots(cpu_gen, T_DECODE, N_SLOTS, P_NONE)
    work = []
    for _ in range(layers):
        layer = []
        for name, (in_dim, outs) in W.DECODE_LAYER.items():
            rn = lambda *s, std=0.02: (torch.randn(*s, generator=gen, device=device) * std).to(torch.bfloat16)  # noqa: E731
            a = [rn(N_SLOTS, RANK, in_dim) for _ in outs]
            b = [rn(N_SLOTS, o, RANK) for o in outs]
            x = rn(T_DECODE, in_dim, std=1.0)
            y = rn(T_DECODE, sum(outs), std=1.0)
            cols = [sum(outs[:i]) for i in range(len(outs))]
            layer.append(dict(name=name, x=x, y=y, a=a, b=b, outs=list(outs), cols=cols))
        work.append(layer)
    return slots, work


def projection_bytes(slots, in_dim, outs):
    active = int(torch.unique(slots[slots >= 0]).numel())
    t_lora = int((slots >= 0).sum())
    n = len(outs)
    return 2 * (active * (n * RANK * in_dim + sum(outs) * RANK) + t_lora * in_dim + 2 * t_lora * sum(outs))


def run_gpu_arm(args):
    import torch.distributed as dist

    from nanovllm_voxcpm_b200 import _native as N
    from nanovllm_voxcpm_b200 import batch_plan as BP
    from nanovllm_voxcpm_b200 import lora as LORA
    from nanovllm_voxcpm_b200 import workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    binding = bind_to_gpu_cpus(local)
    if world > 1:
        _init_dist(device)
    backend = LORA.B200LoRABackend()
    status = backend.availability()
    if not status.available:
        raise RuntimeError(f"B200 LoRA backend unavailable: {status.reason}")

    apply_options(args)
    slots, work = build_gpu_workload(device, args.layers)
    if args.only:
        work = [[p for p in layer if p["name"] == args.only] for layer in work]
    bufs = BP.GraphLoRABuffers.make(T_DECODE, N_SLOTS, device=device)
    bufs.load_plan(BP.build_lora_batch_plan_from_token_to_slot({}, slots.tolist()))
    ctx = bufs.context(T_DECODE)
    meta = LORA.LoRAMetadata(ctx.token_to_slot, ctx.token_indices_sorted_by_slot, ctx.active_slot_ids,
                             ctx.num_tokens_per_slot, ctx.slot_start_offsets, False, ctx.num_active_loras)
    bytes_per_layer = sum(projection_bytes(slots, i, o) for k, (i, o) in W.DECODE_LAYER.items()
                          if args.only in (None, k))
    bytes_per_step = bytes_per_layer * args.layers
    launches_per_step = (1 if args.only else 4) * args.layers

    def step():
        for layer in work:
            for p in layer:
                LORA.launch_add(p["y"], p["x"], p["a"], p["b"], p["outs"], p["cols"], meta, 1.0, impl=N.IMPL_BGMV)

    stream = torch.cuda.Stream(device)
    launch_mode = "eager"
    graph = None
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        if not args.no_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    step()
                launch_mode = "cuda_graph"
            except Exception as exc:  # capture not possible: time eager launches instead
                graph = None
                launch_mode = f"eager (graph capture failed: {type(exc).__name__})"
                torch.cuda.synchronize()
    run_step = graph.replay if graph is not None else step

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    sampler = ClockSampler(local)
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            run_step()
        barrier()
        sampler.start()
        t_wall = time.perf_counter()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(args.steps):
            run_step()
        end.record(stream)
        end.synchronize()
        # keep the sampler alive long enough to take a few readings under load
        while time.perf_counter() - t_wall < 0.6:
            run_step()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        barrier()
    elapsed_ms = start.elapsed_time(end)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    value = bytes_per_step * world / (ms_per_step * 1e-3) / 1e9

    # ---- e2e: public backend call with host buffers ---------------------------------
    e2e = None
    if not args.no_e2e:
        # Host side of a step: per layer ONE pinned staging buffer holding x and y of its projections
        # (x block first, then the y block), mirrored by one device buffer whose slices the LoRA calls
        # use; a layer costs one host->device copy (x and y) and one device->host copy (the y block).
        # All host buffers of a rank are slices of ONE pinned arena (inputs first, then outputs).
        n_in = sum(p["x"].numel() + p["y"].numel() for layer in work for p in layer)
        n_out = sum(p["y"].numel() for layer in work for p in layer)
        arena = torch.empty(n_in + n_out, dtype=torch.bfloat16).pin_memory()
        cursor = {"in": 0, "out": n_in}

        def packed_layer(layer):
            nx = sum(p["x"].numel() for p in layer)
            ny = sum(p["y"].numel() for p in layer)
            dev = torch.empty(nx + ny, dtype=torch.bfloat16, device=device)
            hst = arena[cursor["in"]: cursor["in"] + nx + ny]
            out = arena[cursor["out"]: cursor["out"] + ny]
            cursor["in"] += nx + ny
            cursor["out"] += ny
            views, ox, oy = [], 0, nx
            for p in layer:
                xv = dev[ox: ox + p["x"].numel()].view_as(p["x"])
                yv = dev[oy: oy + p["y"].numel()].view_as(p["y"])
                hst[ox: ox + p["x"].numel()].copy_(p["x"].flatten().cpu())
                hst[oy: oy + p["y"].numel()].copy_(p["y"].flatten().cpu())
                views.append(dict(x=xv, y=yv, ys=list(yv.split(p["outs"], dim=-1)), a=p["a"], b=p["b"]))
                ox += p["x"].numel()
                oy += p["y"].numel()
            return dict(dev=dev, host=hst, out=out, nx=nx, views=views)

        packed = [packed_layer(layer) for layer in work]
        h2d = sum(pl["host"].numel() * 2 for pl in packed)
        d2h = sum(pl["out"].numel() * 2 for pl in packed)
        eager_meta = None
        # Three streams: host->device copies, the LoRA launches, device->host reads, pipelined over the
        # layers; the next step may overwrite a layer's buffer only after its read-back has finished.
        s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        ev_in = [torch.cuda.Event() for _ in packed]
        ev_done = [torch.cuda.Event() for _ in packed]
        ev_out = [torch.cuda.Event() for _ in packed]
        for ev in ev_out:
            ev.record(stream)

        def e2e_step():
            for li, pl in enumerate(packed):
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_out[li])
                    pl["dev"].copy_(pl["host"], non_blocking=True)
                    ev_in[li].record(s_in)
                stream.wait_event(ev_in[li])
                for v in pl["views"]:
                    backend.add_lora(v["ys"], v["x"], v["a"], v["b"], indices=meta.token_to_slot, metadata=meta,
                                     scaling=1.0, y_packed=v["y"])
                ev_done[li].record(stream)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[li])
                    pl["out"].copy_(pl["dev"][pl["nx"]:], non_blocking=True)
                    ev_out[li].record(s_out)

        with torch.cuda.stream(stream):
            for _ in range(min(args.warmup, 3)):
                e2e_step()
            barrier()
            s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n_e2e = max(3, min(args.steps, 10))
            s2.record(stream)
            s_in.wait_event(s2)
            for _ in range(n_e2e):
                e2e_step()
            stream.wait_stream(s_out)  # the last read-back ends the timed region
            e2.record(stream)
            e2.synchronize()
            barrier()
        e2e_ms = s2.elapsed_time(e2)
        if world > 1:
            t = torch.tensor([e2e_ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        del eager_meta
        e2e = {"value": bytes_per_step * world / (e2e_ms / n_e2e * 1e-3) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / n_e2e, "steps": n_e2e,
               # what one rank moves over its host link per second (both directions), and what bound it to its CPUs
               "per_rank_host_link_gbs": (h2d + d2h) / (e2e_ms / n_e2e * 1e-3) / 1e9,
               "per_rank_value": bytes_per_step / (e2e_ms / n_e2e * 1e-3) / 1e9, "cpu_binding": binding}

    # ---- the headline line is complete here; what follows can only add blocks to it ----------------------------
    status_word = N.device_status()
    line = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        per_launch_s = ms_per_step * 1e-3 / launches_per_step
        achieved = bytes_per_step / launches_per_step / per_launch_s / 1e9
        traffic = None
        try:
            with open(os.path.join(ROOT, "profiles", "roofline_traffic.json")) as f:
                traffic = json.load(f).get("bgmv_fused_kernel_bytes_per_launch")
        except Exception:
            pass
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config_dict(args.layers),
            "launch_mode": launch_mode, "gpu_launches": launches_per_step * args.steps,
            "tokens_per_s": T_DECODE * args.layers * world / (ms_per_step * 1e-3),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "peak_kind": f"of {peak_kind}", "kernel": "bgmv_fused_kernel",
                         "us_per_launch": per_launch_s * 1e6, "algorithmic_bytes_per_launch": bytes_per_step / launches_per_step,
                         "frac_of_nominal_8TBs": achieved / 8000.0},
            "clocks": clocks, "device_status": status_word,
        }
        if e2e is not None:
            line["e2e"] = e2e

    # ---- further blocks of the same line (skipped by --no-extras and in tuning runs of a subset) --------------
    extras = {}
    emit = _LineEmitter(line, extras, rank)
    if not args.no_extras and args.only is None and args.layers == N_LAYERS and graph is not None:
        import copy

        # A block that stalls (a rank that left a collective early, a box in trouble) must not cost the headline:
        # after the limit rank 0 prints the line with the blocks it has and every rank leaves.
        emit.arm(args.extras_limit)

        def guarded(fn):
            try:
                return fn()
            except Exception as exc:  # a block that cannot run is reported, the headline stays
                return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}

        def brief(line, keys):
            return {k: line[k] for k in keys if k in line} if "unavailable" not in line else line

        if world == 1:
            # the tensor-core kernels: prefill add (HBM-bound) and fused base GEMM + LoRA (tensor-bound)
            sec = {}
            extras["secondary"] = sec
            for wl in ("prefill", "linear"):
                a2 = copy.copy(args)
                a2.workload, a2.only, a2.steps, a2.warmup = wl, None, 10, 3
                sec[wl] = guarded(lambda a2=a2: brief(run_prefill_arm(a2, emit=False),
                                                      ("metric", "value", "unit", "ms_per_step", "roofline", "us_per_projection",
                                                       "clocks", "cublas_plus_prefill_add_ms_per_step", "lora_tflops")))
            # the incumbent on the same GPU and inputs: the unmodified reference package's own Triton backend
            a3 = copy.copy(args)
            a3.workload, a3.only, a3.steps, a3.warmup = "decode", None, 10, 3
            extras["reference_gpu"] = guarded(lambda: brief(run_reference_gpu_arm(a3, emit=False),
                                                            ("value", "unit", "ms_per_step", "us_per_projection_call", "launch_mode",
                                                             "backend", "unavailable")))
        extras["backbone"] = guarded(lambda: backbone_replicas_block(device, world))
        if world > 1:
            extras["tp"] = guarded(lambda: tp_block(device, world, rank))
        try:
            line_status = N.device_status()
            if rank == 0 and line_status != status_word:
                line["device_status"] = line_status
        except Exception:
            pass
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        r = time_cpu_oracle(steps=40, warmup=3, budget_s=15.0)
        line["cpu_baseline"] = {
            "value": r["gbs"], "unit": "GB/s", "cores": r["cores"], "kind": "port",
            "sample": f"one layer (4 projections, {r['bytes'] / 1e6:.1f} MB algorithmic) x {r['iters']} iterations, "
                      f"fp32 torch CPU per-slot formula, median {r['ms']:.2f} ms",
            # one CPU step is ONE layer; a step of the GPU arm is 24 layers: compare the GB/s, not the step times
            "unit_of_work": "one layer per CPU step (the GPU step above is 24 layers)",
        }
        if not args.no_extras:
            # the same formula on the other two CPU-runnable configurations (bounded samples)
            others = {}
            for key, cfg_name, budget in (("reference_op_T64", "reference_op", 3.0), ("prefill_layer", "prefill", 12.0)):
                q = time_cpu_oracle(steps=20, warmup=2, budget_s=budget, config=cfg_name)
                others[key] = {"value": q["gbs"], "unit": "GB/s", "ms_per_step": q["ms"], "iterations": q["iters"],
                               "algorithmic_mb": q["bytes"] / 1e6}
            line["cpu_baseline"]["other_configs"] = others
    emit.disarm()
    emit()
    if world > 1:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


class _LineEmitter:
    """Prints rank 0's JSON line exactly once: at the normal end, or - if the additional blocks do not finish
    within their limit, or the launcher ends the job because another rank failed - from a watchdog thread /
    the SIGTERM handler, with the blocks that are complete and a note; the process then leaves with status 0."""

    def __init__(self, line, extras, rank):
        import threading

        self.line, self.extras, self.rank = line, extras, rank
        self._lock = threading.Lock()
        self._done = False
        self._timer = None

    def __call__(self, note=None):
        with self._lock:
            if self._done:
                return
            self._done = True
            if self.rank == 0 and self.line is not None:
                out = dict(self.line)
                out.update(self.extras)
                if note:
                    out["extras_note"] = note
                print(json.dumps(out, default=str), flush=True)

    def _bail(self, note):
        self(note)
        sys.stdout.flush()
        os._exit(0)

    def arm(self, limit_s):
        import signal
        import threading

        if limit_s and limit_s > 0:
            # rank 0 speaks first; the other ranks leave a moment later
            delay = limit_s + (0.0 if self.rank == 0 else 5.0)
            self._timer = threading.Timer(delay, self._bail, args=(f"additional blocks cut short after {limit_s:.0f} s",))
            self._timer.daemon = True
            self._timer.start()
        if self.rank == 0:
            try:
                signal.signal(signal.SIGTERM, lambda signum, frame: self._bail("additional blocks cut short: job terminated"))
            except ValueError:  # not the main thread
                pass

    def disarm(self):
        if self._timer is not None:
            self._timer.cancel()
            self._timer = None


# ------------------------------------------------------------------ secondary workloads (prefill kernels)
def run_prefill_arm(args, emit=True):
    """One step = the four multi-LoRA projections of one prefill layer (16 requests, <= 8192 rows, hidden 2048,
    intermediate 6144, ranks 8/16/64 in a rank-64 slab). `prefill`: y += delta through lora_b200_add
    (tcgen05 shrink + tile / run expand), HBM-bound. `linear`: y = x W^T + delta through lora_b200_linear_lora,
    tensor-bound; cuBLAS + the prefill add is timed beside it. Inputs of one layer (> 0.6 GB) exceed L2."""
    from nanovllm_voxcpm_b200 import _native as N
    from nanovllm_voxcpm_b200 import batch_plan as BP
    from nanovllm_voxcpm_b200 import lora as LORA
    from nanovllm_voxcpm_b200 import workloads as W

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise RuntimeError("--workload prefill / linear are single-GPU measurements")
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    names = [args.only] if args.only else list(W.PREFILL_LAYER)
    sets = []
    for k in range(2):  # two independent layer sets, alternated
        layer = []
        for name in names:
            p = W.prefill_projection(name, seed=k)
            gen = torch.Generator().manual_seed(100 + k)
            p.weight = (torch.randn(sum(p.out_sizes), p.x.shape[1], generator=gen) * 0.02).to(torch.bfloat16)
            layer.append((name, p, p.to_device(device)))
        sets.append(layer)
    metas = {}
    for name, p, d in sets[0] + sets[1]:
        ctx = BP.build_lora_context_from_batch_plan(
            BP.build_lora_batch_plan_from_token_to_slot({}, p.token_to_slot.tolist()), device=device)
        metas[id(d)] = LORA.LoRAMetadata(ctx.token_to_slot, ctx.token_indices_sorted_by_slot, ctx.active_slot_ids,
                                         ctx.num_tokens_per_slot, ctx.slot_start_offsets, False, ctx.num_active_loras)
    T = sets[0][0][1].x.shape[0]
    linear = args.workload == "linear"
    outs = {id(d): torch.empty_like(d.y) for layer in sets for _, _, d in layer}

    def launch(d):
        if linear:
            LORA.linear_lora(d.x, d.weight, None, d.a_slabs, d.b_slabs, d.out_sizes, d.col_offsets, d.token_to_slot, 1.0,
                             out=outs[id(d)])
        else:
            LORA.launch_add(d.y, d.x, d.a_slabs, d.b_slabs, d.out_sizes, d.col_offsets, metas[id(d)], 1.0, impl=N.IMPL_SGMV)

    def unfused(d):
        y = torch.mm(d.x, d.weight.t(), out=outs[id(d)])  # cuBLAS into a preallocated output
        LORA.launch_add(y, d.x, d.a_slabs, d.b_slabs, d.out_sizes, d.col_offsets, metas[id(d)], 1.0, impl=N.IMPL_SGMV)

    def timed(fn, reps):
        """ms per call of fn(i); calls i = 0, 1 (the two layer sets) are captured in one CUDA graph and replayed, so
        that the host side of a call (tensor-map encoding, Python) is not part of the number; --no-graph times
        eager launches."""
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if args.no_graph:
            torch.cuda.synchronize()
            s.record()
            for i in range(reps):
                fn(i)
            e.record()
            e.synchronize()
            return s.elapsed_time(e) / reps
        stream = torch.cuda.Stream(device)
        with torch.cuda.stream(stream):
            fn(0), fn(1)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                fn(0), fn(1)
            graph.replay()
            stream.synchronize()
            pairs = max(1, reps // 2)
            s.record(stream)
            for _ in range(pairs):
                graph.replay()
            e.record(stream)
            e.synchronize()
        return s.elapsed_time(e) / (2 * pairs)

    step = lambda i: [launch(d) for _, _, d in sets[i & 1]]  # noqa: E731
    for i in range(max(3, args.warmup)):
        step(i)
    sampler = ClockSampler(0)
    sampler.start()
    t_wall = time.perf_counter()
    ms_per_step = timed(step, args.steps)
    while time.perf_counter() - t_wall < 0.6:
        step(0)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    per_proj = {}
    for j, name in enumerate(names):
        per_proj[name] = timed(lambda i, j=j: launch(sets[i & 1][j][2]), max(args.steps, 10)) * 1e3
    bytes_step = sum(W.algorithmic_bytes(p) for _, p, _ in sets[0])
    lora_flops = 0
    for _, p, _ in sets[0]:
        r_tok = p.ranks[p.token_to_slot.clamp(min=0).long()] * (p.token_to_slot >= 0)
        lora_flops += int(r_tok.sum()) * 2 * (len(p.out_sizes) * p.x.shape[1] + sum(p.out_sizes))
    base_flops = sum(2 * T * p.x.shape[1] * sum(p.out_sizes) for _, p, _ in sets[0])
    hbm_peak, kind = measured_peak()
    line = {"n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"prefill layer: 16 requests, T={T} rows, hidden 2048, intermediate 6144, 16 adapters "
                                   f"ranks 8/16/64 in a rank-64 slab; projections {'+'.join(names)}",
                       "cache_defeat": "inputs larger than L2 (two layer sets of > 0.6 GB alternated)"},
            "us_per_projection": per_proj, "clocks": clocks, "device_status": N.device_status()}
    if linear:
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
            tf_peak, tkind = float(peaks["bf16_tflops"]), "measured burst"
            tf_sustained = float(peaks.get("bf16_tflops_sustained", 0.0)) or None
        except Exception:
            tf_peak, tkind, tf_sustained = 1590.0, "fallback", 1400.0
        for i in range(3):  # cuBLAS handle / heuristics outside the timed region
            [unfused(d) for _, _, d in sets[i & 1]]
        unf = timed(lambda i: [unfused(d) for _, _, d in sets[i & 1]], max(3, args.steps // 2))
        ach = (base_flops + lora_flops) / (ms_per_step * 1e-3) / 1e12
        line.update({"metric": "fused base GEMM + multi-LoRA TFLOP/s (prefill layer, algorithmic flops)", "value": ach,
                     "unit": "TFLOP/s", "gpu_launches": 2 * len(names) * args.steps,
                     "roofline": {"bound": "tensor", "achieved": ach, "peak": tf_peak, "unit": "TFLOP/s",
                                  "frac": ach / tf_peak, "traffic": None, "peak_kind": f"of {tkind}",
                                  "kernel": "tc_tile_kernel", "algorithmic_flops_per_step": base_flops + lora_flops,
                                  # the step runs back to back for longer than a burst; with sw_power_cap active
                                  # the sustained cuBLAS figure is the comparable one
                                  "frac_of_sustained_peak": (ach / tf_sustained) if tf_sustained else None,
                                  "sustained_peak": tf_sustained},
                     "cublas_plus_prefill_add_ms_per_step": unf})
    else:
        ach = bytes_step / (ms_per_step * 1e-3) / 1e9
        line.update({"metric": "multi-LoRA linear GB/s (prefill SGMV, algorithmic bytes)", "value": ach, "unit": "GB/s",
                     "gpu_launches": 2 * len(names) * args.steps,
                     "roofline": {"bound": "hbm", "achieved": ach, "peak": hbm_peak, "unit": "GB/s", "frac": ach / hbm_peak,
                                  "traffic": None, "peak_kind": f"of {kind}",
                                  "kernel": "sgmv_shrink_kernel + tc_tile_kernel",
                                  "algorithmic_bytes_per_step": bytes_step},
                     "lora_tflops": lora_flops / (ms_per_step * 1e-3) / 1e12})
    if emit:
        print(json.dumps(line))
    return line


# ------------------------------------------------------------------ the reference's own GPU backend
def run_reference_gpu_arm(args, emit=True):
    """Times `get_backend().add_lora` of the UNMODIFIED reference package (installed from its source tree into
    baseline/_ref; nothing of this library on the path) on the decode or prefill workload of this file, eagerly
    and, for decode, inside a CUDA graph exactly as its runner replays it. Prints one JSON line."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if int(os.environ.get("RANK", "0")) != 0:
        return
    try:
        if not os.path.isdir(os.path.join(ref_root, "nanovllm_voxcpm")):
            raise RuntimeError("baseline/_ref holds no install of the reference")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
        sys.path.insert(0, ref_root)
        import nanovllm_voxcpm.lora as RL

        status = RL.get_availability()
        if not status.available:
            raise RuntimeError(f"reference backend unavailable: {status.reason}")
        backend = RL.get_backend()
    except Exception as exc:
        line = {"impl": "reference-gpu", "unavailable": f"{type(exc).__name__}: {exc}"[:300]}
        if emit:
            print(json.dumps(line))
        return line
    from nanovllm_voxcpm_b200 import batch_plan as BP
    from nanovllm_voxcpm_b200 import workloads as W

    device = torch.device("cuda", torch.cuda.current_device())
    decode = args.workload == "decode"
    if decode:
        slots, work = build_gpu_workload(device, args.layers)
        bufs = BP.GraphLoRABuffers.make(T_DECODE, N_SLOTS, device=device)
        bufs.load_plan(BP.build_lora_batch_plan_from_token_to_slot({}, slots.tolist()))
        ctx = bufs.context(T_DECODE)
        if args.only:
            work = [[p for p in layer if p["name"] == args.only] for layer in work]
        bytes_step = sum(projection_bytes(slots, i, o) for k, (i, o) in W.DECODE_LAYER.items()
                         if args.only in (None, k)) * args.layers
        meta = RL.LoRAMetadata(ctx.token_to_slot, ctx.token_indices_sorted_by_slot, ctx.active_slot_ids,
                               ctx.num_tokens_per_slot, ctx.slot_start_offsets, False, ctx.num_active_loras)
        metas = None
    else:
        names = [args.only] if args.only else list(W.PREFILL_LAYER)
        work, metas, bytes_step = [], {}, 0
        for k in range(2):
            layer = []
            for name in names:
                p = W.prefill_projection(name, seed=k)
                d = p.to_device(device)
                c = BP.build_lora_context_from_batch_plan(
                    BP.build_lora_batch_plan_from_token_to_slot({}, p.token_to_slot.tolist()), device=device)
                item = dict(name=name, x=d.x, y=d.y, a=d.a_slabs, b=d.b_slabs, outs=list(d.out_sizes))
                metas[id(item)] = RL.LoRAMetadata(c.token_to_slot, c.token_indices_sorted_by_slot, c.active_slot_ids,
                                                  c.num_tokens_per_slot, c.slot_start_offsets, False, c.num_active_loras)
                layer.append(item)
                if k == 0:
                    bytes_step += W.algorithmic_bytes(p)
            work.append(layer)
        meta = None

    def step(i=None):
        layers = work if decode else [work[(i or 0) & 1]]
        for layer in layers:
            for p in layer:
                m = meta if decode else metas[id(p)]
                backend.add_lora(list(p["y"].split(p["outs"], dim=-1)), p["x"], p["a"], p["b"],
                                 indices=m.token_to_slot, metadata=m, scaling=1.0, y_packed=p["y"])

    stream = torch.cuda.Stream(device)
    mode = "eager"
    with torch.inference_mode(), torch.cuda.stream(stream):
        for i in range(max(3, args.warmup)):  # Triton compiles and autotunes here
            step(i)
        stream.synchronize()
        run = step
        if decode and not args.no_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    step()
                run = lambda i=None: graph.replay()  # noqa: E731
                mode = "cuda_graph"
            except Exception as exc:
                mode = f"eager (graph capture failed: {type(exc).__name__})"
                torch.cuda.synchronize()
        for i in range(3):
            run(i)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream.synchronize()
        s.record(stream)
        for i in range(args.steps):
            run(i)
        e.record(stream)
        e.synchronize()
    ms = s.elapsed_time(e) / args.steps
    value = bytes_step / (ms * 1e-3) / 1e9
    nproj = sum(len(layer) for layer in work) if decode else len(work[0])
    line = {
        "impl": "reference-gpu", "metric": METRIC if decode else "multi-LoRA linear GB/s (prefill SGMV, algorithmic bytes)",
        "value": value, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_dict(args.layers) if decode else {"workload": "prefill layer (see --workload prefill)"},
        "launch_mode": mode, "us_per_projection_call": ms * 1e3 / nproj,
        "backend": type(backend).__name__,
    }
    if emit:
        print(json.dumps(line))
    return line


# ------------------------------------------------------------------ whole decoder step around the LoRA linears
def run_backbone_arm(args):
    """Random-init 24-layer decoder (hidden 1024, 16 q / 2 kv heads x 64, intermediate 4096), 64 requests with
    prompts of 128-512 tokens, 128 resident rank-32 adapters (4.3 GB of slabs), adapter per request ~ Zipf(1.1):
    one prefill pass over all prompts, then decode steps of one token per request replayed from a CUDA graph.
    Attention / norms / RoPE / activation are library code (flash_attn, torch); timed with and without adapters."""
    from nanovllm_voxcpm_b200 import _native as N
    from nanovllm_voxcpm_b200 import backbone as BB

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise RuntimeError("--workload backbone is a single-GPU measurement")
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    apply_options(args)
    cfg = BB.DecoderConfig(num_layers=args.layers)
    n_req, decode_steps = 64, args.steps if args.steps != 20 else 512
    gen = torch.Generator().manual_seed(0)
    prompts = torch.randint(128, 513, (n_req,), generator=gen).tolist()
    work = BB.BackboneWorkload(prompts, BB.zipf_adapters(n_req, cfg.max_loras, 1.1, seed=0), decode_steps)
    with torch.device(device):
        model = BB.Decoder(cfg).to(torch.bfloat16)
    model.init_random_(0)
    model.fill_adapter_slots_(cfg.max_loras, cfg.max_lora_rank, seed=1)
    model.fused_glue = args.glue == "fused" and args.impl == "b200"
    from nanovllm_voxcpm_b200 import layers as L_

    L_.LORA_FIRST = args.lora_order == "first" and args.impl == "b200"
    backend_name = "B200LoRABackend"
    if args.impl == "reference-gpu":
        # same decoder, same layers, but every LoRA call goes to the unmodified reference's own GPU backend
        try:
            sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
            import nanovllm_voxcpm.lora as RL
            from nanovllm_voxcpm_b200 import lora as LORA

            status = RL.get_availability()
            if not status.available:
                raise RuntimeError(f"reference backend unavailable: {status.reason}")
            LORA.set_backend_for_testing(RL.get_backend())
            backend_name = type(RL.get_backend()).__name__
        except Exception as exc:
            print(json.dumps({"impl": "reference-gpu", "unavailable": f"{type(exc).__name__}: {exc}"[:300]}))
            return
    result = {}
    for tag, use_lora in (("lora", True), ("base", False)):
        runner = BB.BackboneRunner(model, work, use_lora=use_lora)
        runner.prefill()  # warm-up (cuBLAS / flash_attn set-up, scratch allocation)
        p_tok, p_ms = runner.prefill()
        d_tok, d_ms, mode = runner.decode(decode_steps, use_graph=not args.no_graph)
        result[tag] = {"prefill_tokens_per_s": p_tok / (p_ms * 1e-3), "prefill_ms": p_ms, "prefill_tokens": p_tok,
                       "decode_tokens_per_s": d_tok / (d_ms * 1e-3), "decode_ms_per_step": d_ms / decode_steps,
                       "launch_mode": mode}
    lora, base = result["lora"], result["base"]
    print(json.dumps({
        "metric": "decoder backbone decode tokens/s with 128 resident adapters (64 requests x 1 token per step)",
        "value": lora["decode_tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": decode_steps, "warmup": 3,
        "ms_per_step": lora["decode_ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"decoder backbone: {cfg.num_layers} layers, hidden 1024, 16/2 heads x 64, intermediate 4096, "
                               f"{n_req} requests, prompts 128-512 (sum {sum(prompts)}), {decode_steps} decode steps, "
                               f"{cfg.max_loras} adapters rank {cfg.max_lora_rank}, Zipf(1.1) "
                               f"({len(set(work.adapter_of_request))} distinct in the batch), paged KV block 256"},
        "with_adapters": lora, "without_adapters": base,
        "adapter_overhead": {"decode": base["decode_tokens_per_s"] / lora["decode_tokens_per_s"],
                             "prefill": base["prefill_tokens_per_s"] / lora["prefill_tokens_per_s"]},
        "device_status": N.device_status(), "impl": args.impl, "lora_backend": backend_name,
        "glue": "fused kernels" if model.fused_glue else "torch ops",
        "lora_order": "first" if L_.LORA_FIRST else "after",
    }))


# ------------------------------------------------------------------ glue kernels between the projections
def run_glue_arm(args):
    """The three single-launch glue kernels on a prefill batch (8192 rows; hidden 1024, 16 q / 2 kv heads x 64,
    intermediate 4096), each against the chain of torch ops it replaces. Every call works on the next of several
    buffer sets that together exceed L2, so rows come from HBM; timed with CUDA events."""
    from nanovllm_voxcpm_b200 import _native as N
    from nanovllm_voxcpm_b200 import backbone as BB
    from nanovllm_voxcpm_b200 import glue as G

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(0)
    dev, dt = torch.device("cuda", 0), torch.bfloat16
    T, H, I, heads, kvh, D = 8192, 1024, 4096, 16, 2, 64
    peak, peak_kind = measured_peak()
    reps, warm = max(args.steps, 20), max(args.warmup, 3)

    def timed(fn, n_sets):
        """us per call; one pass over all buffer sets is captured in a CUDA graph so that the host-side cost of
        a call (tens of microseconds of Python) does not hide kernels that take about as long."""
        stream = torch.cuda.Stream(dev)
        with torch.cuda.stream(stream):
            for i in range(max(warm, n_sets)):
                fn(i % n_sets)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(n_sets):
                    fn(i)
            for _ in range(warm):
                graph.replay()
            stream.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(stream)
            for _ in range(reps):
                graph.replay()
            e.record(stream)
            e.synchronize()
        return s.elapsed_time(e) / (reps * n_sets) * 1e3

    out = {}
    # residual add + RMSNorm: reads x, residual; writes hidden, normed
    n = 6
    xs = [torch.randn(T, H, device=dev).to(dt) for _ in range(n)]
    rs = [torch.randn(T, H, device=dev).to(dt) for _ in range(n)]
    hs, ns = [torch.empty_like(x) for x in xs], [torch.empty_like(x) for x in xs]
    w = torch.ones(H, device=dev, dtype=dt)

    def torch_norm(i):
        h = rs[i] + xs[i]
        BB._rms_norm(h, w, 1e-6)

    nbytes = 4 * T * H * 2
    us, ref_us = timed(lambda i: G.add_rms_norm(xs[i], rs[i], w, 1e-6, out=ns[i], hidden_out=hs[i]), n), timed(torch_norm, n)
    out["add_rmsnorm"] = {"us": us, "gbs": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / peak, "torch_ops_us": ref_us}
    del xs, rs, hs, ns
    # RoPE + cache store: reads q, k, v rows, writes q, k rows and the k, v cache rows
    n = 10
    width = (heads + 2 * kvh) * D
    qkvs = [torch.randn(T, width, device=dev).to(dt) for _ in range(n)]
    pos = torch.randint(0, 4096, (T,), device=dev)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    freqs = torch.outer(torch.arange(4096, dtype=torch.float32), inv)
    cos, sin = freqs.cos().to(dev), freqs.sin().to(dev)
    kc, vc = torch.zeros(T, kvh, D, device=dev, dtype=dt), torch.zeros(T, kvh, D, device=dev, dtype=dt)
    slot = torch.randperm(T, device=dev)
    slot32 = slot.to(torch.int32)

    def torch_rope(i):
        q, k, v = qkvs[i].split([heads * D, kvh * D, kvh * D], dim=-1)
        c, s = cos[pos].unsqueeze(1), sin[pos].unsqueeze(1)
        BB._rope(q.view(T, heads, D), c, s)
        kk = BB._rope(k.view(T, kvh, D), c, s)
        kc.index_copy_(0, slot, kk)
        vc.index_copy_(0, slot, v.reshape(T, kvh, D))

    nbytes = T * (width + (heads + kvh) * D + 2 * kvh * D) * 2
    us = timed(lambda i: G.rope_kv_store(qkvs[i], heads, kvh, D, positions=pos, cos=cos, sin=sin, k_cache=kc, v_cache=vc,
                                         slot_mapping=slot32), n)
    out["rope_kv_store"] = {"us": us, "gbs": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / peak, "torch_ops_us": timed(torch_rope, n)}
    del qkvs
    # SiLU * up: reads gate | up, writes the product
    n = 2
    gus = [torch.randn(T, 2 * I, device=dev).to(dt) for _ in range(n)]
    outs = [torch.empty(T, I, device=dev, dtype=dt) for _ in range(n)]

    def torch_silu(i):
        g, u = gus[i].chunk(2, dim=-1)
        torch.nn.functional.silu(g) * u

    nbytes = 3 * T * I * 2
    us = timed(lambda i: G.silu_and_mul(gus[i], out=outs[i]), n)
    out["silu_mul"] = {"us": us, "gbs": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / peak, "torch_ops_us": timed(torch_silu, n)}
    total = sum(v["us"] for v in out.values())
    total_bytes = sum(v["gbs"] * v["us"] * 1e3 for v in out.values())
    print(json.dumps({
        "metric": "decoder-layer glue GB/s (residual add + RMSNorm, RoPE + cache store, SiLU * up; algorithmic bytes)",
        "value": total_bytes / total / 1e3, "unit": "GB/s", "n_gpus": 1, "steps": reps, "warmup": warm,
        "ms_per_step": total * 1e-3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"glue of one layer on {T} rows: hidden {H}, {heads}/{kvh} heads x {D}, intermediate {I}",
                   "cache_defeat": "buffer sets rotated, larger than L2 together"},
        "roofline": {"bound": "hbm", "achieved": total_bytes / total / 1e3, "peak": peak, "unit": "GB/s",
                     "frac": total_bytes / total / 1e3 / peak, "traffic": None, "peak_kind": peak_kind},
        "kernels": out, "gpu_launches": (6 + 10 + 2) * reps, "device_status": N.device_status(),
    }))


# ------------------------------------------------------------------ adapter admission (checkpoint -> resident slot)
def run_admission_arm(args):
    """One adapter (rank 32, every projection of a 24-layer decoder, fp32 payload of ~68 MB) admitted into a slot:
    `SlotLoader.load_slot` (one descriptor table + the payload's pinned arena copied as it lies, one kernel) against
    the module-by-module procedure of the reference's runner (per module: host->device copy per tensor, clear, copy
    the used rows / columns, scale B). Wall clock per admission, device idle before and after."""
    import tempfile

    from nanovllm_voxcpm_b200 import _native as N
    from nanovllm_voxcpm_b200 import adapter_checkpoint as AC
    from nanovllm_voxcpm_b200 import backbone as BB
    from nanovllm_voxcpm_b200 import layers as L
    from nanovllm_voxcpm_b200.slot_loader import SlotLoader

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise RuntimeError("--workload admission is a single-GPU measurement")
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    cfg = BB.DecoderConfig(num_layers=args.layers, max_loras=8)
    with torch.device(device):
        model = BB.Decoder(cfg).to(torch.bfloat16)
    modules = {n: m for n, m in model.named_modules() if isinstance(m, L._LORA_LAYER_TYPES)}
    gen = torch.Generator().manual_seed(0)
    rank, tensors = cfg.max_lora_rank, {}
    unpack = {"qkv_proj": ("q_proj", "k_proj", "v_proj"), "gate_up_proj": ("gate_proj", "up_proj")}
    for name, m in modules.items():
        parent, _, leaf = name.rpartition(".")
        for proj, a_slab, b_slab in zip(unpack.get(leaf, (leaf,)), m._a_slices(), m._b_slices()):
            tensors[f"{parent}.{proj}.lora_A"] = torch.randn(rank, a_slab.size(2), generator=gen) * 0.05
            tensors[f"{parent}.{proj}.lora_B"] = torch.randn(b_slab.size(1), rank, generator=gen) * 0.05
    with tempfile.TemporaryDirectory() as root:
        path = AC.save_lora_checkpoint(os.path.join(root, "adapter"), tensors, rank=rank, alpha=2.0 * rank)
        AC.load_lora_checkpoint(str(path))
        t0 = time.perf_counter()
        payload = AC.load_lora_checkpoint(str(path))
        read_ms = (time.perf_counter() - t0) * 1e3
    payload_bytes = sum(t.numel() * 4 for t in tensors.values())
    loader = SlotLoader(model)
    loaded = {}

    def by_module(slot):
        for name in loaded.get(slot, []):
            modules[name].clear_slot_lora(slot)
        for name, mp in payload.modules.items():
            b = mp.lora_b
            modules[name].set_slot_lora(slot, mp.lora_a.to(device="cuda", non_blocking=True),
                                        [t.to(device="cuda", non_blocking=True) for t in b] if isinstance(b, list)
                                        else b.to(device="cuda", non_blocking=True), mp.effective_rank, mp.scaling)
        loaded[slot] = list(payload.modules)

    def wall(fn, reps, warm):
        for i in range(warm):
            fn(i % cfg.max_loras)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(reps):
            fn(i % cfg.max_loras)
            torch.cuda.synchronize()
        return (time.perf_counter() - t0) / reps * 1e3

    reps, warm = args.steps, max(args.warmup, 3)
    one_launch_ms = wall(lambda s: loader.load_slot(s, payload), reps, warm)
    slabs = {n: [t.detach().clone() for t in (*m._a_slices(), *m._b_slices())] for n, m in modules.items()}
    per_module_ms = wall(by_module, reps, warm)
    same = all(torch.equal(a, b) for n, m in modules.items() for a, b in zip(slabs[n], (*m._a_slices(), *m._b_slices())))
    print(json.dumps({
        "metric": "adapter admission ms (checkpoint payload on the host -> resident slot)", "value": one_launch_ms,
        "unit": "ms", "n_gpus": 1, "steps": reps, "warmup": warm, "ms_per_step": one_launch_ms, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"one rank-{rank} adapter over {len(modules)} modules of a {cfg.num_layers}-layer decoder, "
                               f"{payload_bytes / 1e6:.1f} MB fp32 payload, bf16 slabs"},
        "module_by_module_ms": per_module_ms, "speedup": per_module_ms / one_launch_ms,
        "h2d_gbs": payload_bytes / (one_launch_ms * 1e-3) / 1e9, "checkpoint_read_ms": read_ms,
        "slabs_identical": bool(same), "gpu_launches": reps, "device_status": N.device_status(),
    }))


# ------------------------------------------------------------------ tensor-parallel row-parallel projection
def run_tp_arm(args):
    """Launched with torchrun on N >= 2 GPUs: the `down` projection of an 8-GPU-class layer (hidden 4096,
    intermediate 14336, rank 64) as a row-parallel layer over N ranks, decode batch of 512 rows, in the three
    exchange modes, and the exchange of the [T, r] partials alone (peer-memory kernel vs NCCL)."""
    import torch.distributed as dist

    from nanovllm_voxcpm_b200 import _native as N
    from nanovllm_voxcpm_b200 import context as CTX
    from nanovllm_voxcpm_b200 import layers as L
    from nanovllm_voxcpm_b200.tp_exchange import TpExchange

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise RuntimeError("--workload tp needs torchrun with at least two ranks")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    T, hidden, inter, S, r = 512, 4096, 14336, 32, 64
    ex = TpExchange(capacity=8704 * r)

    def timed(fn, reps):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(reps):
            fn()
        e.record()
        e.synchronize()
        t = torch.tensor([s.elapsed_time(e) / reps * 1e3], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    exchange = {}
    for name, rows in (("decode_512x64", 512), ("prefill_8704x64", 8704)):
        part = torch.randn(rows * r, device=device)
        exchange[name] = {"peer_kernel_us": timed(lambda: ex.all_reduce_(part), 200),
                          "nccl_us": timed(lambda: dist.all_reduce(part), 200), "bytes": rows * r * 4}
    gen = torch.Generator().manual_seed(0)
    slots = torch.randint(-1, S, (T,), generator=gen, dtype=torch.int32).to(device)
    CTX.set_lora_context(CTX.build_lora_context_from_token_to_slot(slots))
    x = torch.randn(T, inter // world, device=device).to(torch.bfloat16)
    layer_us = {}
    for mode in ("partial_y", "allreduce_tmp", "peer_exchange"):
        layer = L.LoRARowParallelLinear(inter, hidden, max_loras=S, max_lora_rank=r, lora_tp_mode=mode).to(device, torch.bfloat16)
        layer.tp_exchange = ex
        with torch.no_grad():
            layer.weight.normal_(0, 0.02)
            layer.lora_A.normal_(0, 0.02)
            layer.lora_B.normal_(0, 0.02)
        for s in range(S):
            layer._effective_lora_rank_values[s] = r
        with torch.inference_mode():
            layer_us[mode] = timed(lambda: layer(x), 100)
        del layer
    status = N.device_status()
    if rank == 0:
        print(json.dumps({
            "metric": "row-parallel multi-LoRA projection us per call (tensor parallel)", "value": layer_us["peer_exchange"],
            "unit": "us", "n_gpus": world, "steps": 100, "warmup": 5, "ms_per_step": layer_us["peer_exchange"] * 1e-3,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"down projection {inter} -> {hidden} sharded over {world} ranks, {T} rows, {S} adapters rank {r}"},
            "layer_us_by_mode": layer_us, "exchange_us": exchange, "device_status": status,
        }))
    dist.destroy_process_group()


# ------------------------------------------------------------------ 8-GPU class decoder (config 5) and multi-GPU blocks
CONFIG5 = dict(hidden_size=4096, num_heads=32, num_kv_heads=8, head_dim=128, intermediate_size=14336, max_lora_rank=64)
N_REGISTERED_5, N_DECODE_5, PREFILL_LENS_5 = 1024, 512, [1024] * 8


def _ranks():
    return int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))


def _init_dist(device):
    """NCCL process group for the plumbing (NVLS off: in-switch reduction is not needed by this path, and the
    exchange buffers of this library are never bound to a multicast object)."""
    import torch.distributed as dist

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=device)
    return dist


def _max_over_ranks(value, device, world):
    if world == 1:
        return float(value)
    import torch.distributed as dist

    t = torch.tensor([float(value)], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _replica_layers(on: bool):
    """Request-level replicas under torchrun: every rank builds the WHOLE model (the layers must not see the
    process group as a tensor-parallel group)."""
    from nanovllm_voxcpm_b200 import layers as L

    if on:
        L._get_world_size, L._get_rank = (lambda: 1), (lambda: 0)
    else:
        from nanovllm_voxcpm_b200.distributed import get_tp_rank, get_tp_world_size

        L._get_world_size, L._get_rank = get_tp_world_size, get_tp_rank


def measure_backbone_replica(device, n_layers=24, decode_steps=128):
    """Config-4 decoder step (24 layers, hidden 1024, 64 requests, 128 resident rank-32 adapters, Zipf) on this GPU:
    one prefill pass over all prompts, then graph-replayed decode steps. Returns tokens and device milliseconds."""
    from nanovllm_voxcpm_b200 import backbone as BB
    from nanovllm_voxcpm_b200 import layers as L_

    cfg = BB.DecoderConfig(num_layers=n_layers)
    gen = torch.Generator().manual_seed(0)
    prompts = torch.randint(128, 513, (64,), generator=gen).tolist()
    work = BB.BackboneWorkload(prompts, BB.zipf_adapters(64, cfg.max_loras, 1.1, seed=0), decode_steps)
    with torch.device(device):
        model = BB.Decoder(cfg).to(torch.bfloat16)
    model.init_random_(0)
    model.fill_adapter_slots_(cfg.max_loras, cfg.max_lora_rank, seed=1)
    model.fused_glue = True
    L_.LORA_FIRST = True
    try:
        runner = BB.BackboneRunner(model, work, use_lora=True)
        runner.prefill()
        p_tok, p_ms = runner.prefill()
        d_tok, d_ms, mode = runner.decode(decode_steps, use_graph=True)
    finally:
        L_.LORA_FIRST = False
    del runner, model
    torch.cuda.empty_cache()
    return {"prefill_tokens": p_tok, "prefill_ms": p_ms, "decode_tokens": d_tok, "decode_ms": d_ms, "launch_mode": mode,
            "decode_steps": decode_steps}


def backbone_replicas_block(device, world):
    """The metric's second half: the config-4 decoder step as `world` request-level replicas (one per GPU, no
    data-path collective): tokens of all ranks / the slowest rank's device time."""
    _replica_layers(True)
    try:
        r = measure_backbone_replica(device)
    finally:
        _replica_layers(False)
    p_ms = _max_over_ranks(r["prefill_ms"], device, world)
    d_ms = _max_over_ranks(r["decode_ms"], device, world)
    return {"parallelism": f"{world} replicas", "workload": "24-layer decoder, hidden 1024, 64 requests per replica, prompts 128-512, "
            f"{r['decode_steps']} decode steps, 128 resident adapters rank 32, Zipf(1.1)",
            "decode_tokens_per_s": r["decode_tokens"] * world / (d_ms * 1e-3),
            "prefill_tokens_per_s": r["prefill_tokens"] * world / (p_ms * 1e-3),
            "decode_ms_per_step": d_ms / r["decode_steps"], "prefill_ms": p_ms, "launch_mode": r["launch_mode"]}


def _config5_requests(resident_slots):
    """Adapter of each request of the step (512 decode requests + 8 prompts): ids ~ Zipf(1.1) over the 1024
    registered adapters, admitted into the resident slots in order of first use; requests whose adapter would not
    fit (more distinct adapters than slots) share the slot id modulo the slot count."""
    from nanovllm_voxcpm_b200 import backbone as BB

    ids = BB.zipf_adapters(N_DECODE_5 + len(PREFILL_LENS_5), N_REGISTERED_5, 1.1, seed=0)
    slot_of, overflow = {}, 0
    for a in ids:
        if a not in slot_of:
            if len(slot_of) < resident_slots:
                slot_of[a] = len(slot_of)
            else:
                slot_of[a] = a % resident_slots
                overflow += 1
    slots = [slot_of[a] for a in ids]
    return slots[:N_DECODE_5], slots[N_DECODE_5:], len(set(ids)), overflow


def measure_config5(device, n_layers, slab_budget_gb, iters, use_lora=True):
    """One mixed step (512 decode rows + an 8192-token prefill chunk) of the 8-GPU class decoder on this rank's
    share of the model (the layers shard themselves by the tensor-parallel world they see)."""
    from nanovllm_voxcpm_b200 import backbone as BB
    from nanovllm_voxcpm_b200 import layers as L

    tp = L._get_world_size()
    mode = "peer_exchange" if tp > 1 else "partial_y"
    with torch.device("meta"):
        probe = BB.Decoder(BB.DecoderConfig(num_layers=1, max_loras=1, lora_tp_mode=mode, **CONFIG5))
    per_slot = sum(t.numel() for m in L.iter_lora_modules(probe) for t in (*m._a_slices(), *m._b_slices())) * 2 * n_layers
    slots = int(max(8, min(N_REGISTERED_5, slab_budget_gb * 1e9 // per_slot)))
    cfg = BB.DecoderConfig(num_layers=n_layers, max_loras=slots, lora_tp_mode=mode, **CONFIG5)
    with torch.device(device):
        model = BB.Decoder(cfg).to(torch.bfloat16)
    model.init_random_(0)
    model.fill_adapter_slots_(slots, cfg.max_lora_rank, seed=1)
    model.fused_glue = True
    exchange = None
    if tp > 1:
        from nanovllm_voxcpm_b200.tp_exchange import TpExchange

        exchange = TpExchange(capacity=(N_DECODE_5 + sum(PREFILL_LENS_5)) * cfg.max_lora_rank)
        model.attach_tp_exchange(exchange)
    dec, pre, distinct, overflow = _config5_requests(slots)
    tokens, ms, _ = BB.time_mixed_step(model, N_DECODE_5, PREFILL_LENS_5, dec, pre, iters=iters, use_lora=use_lora)
    info = {"resident_slots": slots, "slab_gb_per_gpu": per_slot * slots / 1e9, "distinct_adapters_in_step": distinct,
            "requests_sharing_a_slot": overflow, "lora_tp_mode": mode}
    return tokens, ms, info, model, exchange


def run_backbone5_arm(args):
    """BASELINE config 5: random-init 32-layer decoder, hidden 4096, 32 / 8 heads x 128, intermediate 14336, bf16;
    1024 registered rank-64 adapters, a step of 512 decode sequences + one 8192-token prefill chunk. Under torchrun
    the N ranks form one tensor-parallel group (`--parallelism tp`, default) or N request-level replicas
    (`--parallelism replicas`)."""
    from nanovllm_voxcpm_b200 import _native as N

    world, rank, local = _ranks()
    torch.cuda.set_device(local)
    apply_options(args)
    device = torch.device("cuda", local)
    if world > 1:
        _init_dist(device)
    replicas = world > 1 and args.parallelism == "replicas"
    _replica_layers(replicas)
    tp = 1 if replicas or world == 1 else world
    iters = max(3, min(args.steps, 10))
    tokens, ms, info, model, exchange = measure_config5(device, args.layers if args.layers != N_LAYERS else 32,
                                                        args.slab_gb, iters)
    base_tokens, base_ms = tokens, None
    if not args.no_base:
        from nanovllm_voxcpm_b200 import backbone as BB

        dec, pre, _, _ = _config5_requests(info["resident_slots"])
        _, base_ms, _ = BB.time_mixed_step(model, N_DECODE_5, PREFILL_LENS_5, dec, pre, iters=iters, use_lora=False)
        base_ms = _max_over_ranks(base_ms, device, world)
    ms = _max_over_ranks(ms, device, world)
    n_rep = world if replicas else 1
    line = {
        "metric": "decoder backbone tokens/s, 8-GPU class model (512 decode rows + 8192-token prefill chunk per step)",
        "value": tokens * n_rep / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": iters, "warmup": 2,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak" if replicas else "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{model.cfg.num_layers}-layer decoder, hidden 4096, 32/8 heads x 128, intermediate 14336; "
                               f"{N_REGISTERED_5} registered adapters rank 64; step = {N_DECODE_5} decode rows + "
                               f"{sum(PREFILL_LENS_5)}-token prefill chunk ({len(PREFILL_LENS_5)} prompts)",
                   "parallelism": f"{world} replicas x tp1" if replicas else f"tp{tp}",
                   "residency": "adapters are admitted into the resident slots in order of first use (LRU through SlotLoader "
                                "in a serving loop); the step's adapters are resident before the timed region"},
        **info, "device_status": N.device_status(),
    }
    if base_ms is not None:
        line["without_adapters_ms_per_step"] = base_ms
        line["adapter_overhead"] = ms / base_ms
    if exchange is not None:
        line["exchange_us"] = _exchange_times(exchange, device, model.cfg.max_lora_rank, model.cfg.hidden_size)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


def _exchange_times(exchange, device, r, hidden):
    """[T, r] exchange of the row-parallel layers: the peer-memory kernel against NCCL for the decode rows (fp32), NCCL
    for the prefill chunk (bf16), and the [T, hidden] sum of the base output that every row-parallel layer pays anyway."""
    import torch.distributed as dist

    def timed(fn, reps=50):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(reps):
            fn()
        e.record()
        e.synchronize()
        return _max_over_ranks(s.elapsed_time(e) / reps * 1e3, device, dist.get_world_size())

    T = N_DECODE_5 + sum(PREFILL_LENS_5)
    dec = torch.randn(N_DECODE_5 * r, device=device)
    pre = torch.randn(sum(PREFILL_LENS_5), r, device=device).to(torch.bfloat16)
    full = torch.randn(T, hidden, device=device).to(torch.bfloat16)
    return {"decode_rows_[512,r]_fp32": {"bytes": dec.numel() * 4, "peer_kernel_us": timed(lambda: exchange.all_reduce_(dec)),
                                         "nccl_us": timed(lambda: dist.all_reduce(dec))},
            "prefill_rows_[8192,r]_bf16": {"bytes": pre.numel() * 2, "nccl_us": timed(lambda: dist.all_reduce(pre))},
            "base_output_[T,hidden]_bf16": {"bytes": full.numel() * 2, "nccl_us": timed(lambda: dist.all_reduce(full), 20)}}


def tp_block(device, world, rank):
    """Tensor-parallel block of the N-GPU line: (1) parity of a small decoder under TP = N against the same decoder
    on one GPU (rank 0), same seeded weights and adapters, a mixed step; (2) an 8-layer slice of the 8-GPU class
    decoder under TP = N: tokens/s of the mixed step and the exchange times."""
    from nanovllm_voxcpm_b200 import backbone as BB
    from nanovllm_voxcpm_b200.tp_exchange import TpExchange

    # ---- (1) parity on a small case
    small = dict(hidden_size=512, num_heads=8, num_kv_heads=8, head_dim=64, intermediate_size=1024, num_layers=2,
                 max_loras=4, max_lora_rank=32, max_position=1024)
    gen = torch.Generator().manual_seed(5)
    n_dec, lens = 16, [300, 212, 130]
    dec = torch.randint(-1, 4, (n_dec,), generator=gen).tolist()
    pre = [0, 3, 1]

    def run_small(mode):
        with torch.device(device):
            m = BB.Decoder(BB.DecoderConfig(lora_tp_mode=mode, **small)).to(torch.bfloat16)
        m.load_full_random_(4, 32, seed=9, std=0.05)
        m.fused_glue = True
        if mode == "peer_exchange":
            m.attach_tp_exchange(TpExchange(capacity=(n_dec + sum(lens)) * 32))
        return BB.time_mixed_step(m, n_dec, lens, dec, pre, context_len=40, iters=1, warmup=1)[2].float()

    out_tp = run_small("peer_exchange")
    parity, parity_detail = "ok", None
    if rank == 0:
        _replica_layers(True)
        try:
            out_1 = run_small("partial_y")
        finally:
            _replica_layers(False)
        err, ref_max = float((out_tp - out_1).abs().max()), float(out_1.abs().max())
        # two bf16 decoder layers summed in another order per rank count: 6e-2 absolute plus 1 % of the largest
        # output (one bf16 step at that magnitude), the bound the tests use for bf16 stacks
        parity = "ok" if err <= 6e-2 + 1e-2 * ref_max and ref_max > 0.1 else f"max-abs difference {err:.3g} (largest output {ref_max:.3g})"
        parity_detail = {"max_abs_difference": err, "largest_output": ref_max}
    # ---- (2) the 8-GPU class layers under TP = N
    tokens, ms, info, model, exchange = measure_config5(device, 8, 40.0, 3)
    ms = _max_over_ranks(ms, device, world)
    block = {"parallelism": f"tp{world}", "tp_parity": parity, "tp_parity_detail": parity_detail,
             "workload": "8 layers of the 8-GPU class decoder (hidden 4096, 32/8 heads x 128, intermediate 14336), "
                         f"{N_DECODE_5} decode rows + {sum(PREFILL_LENS_5)}-token prefill chunk per step",
             "tokens_per_s": tokens / (ms * 1e-3), "ms_per_step": ms, **info,
             "exchange_us": _exchange_times(exchange, device, model.cfg.max_lora_rank, model.cfg.hidden_size)}
    del model
    torch.cuda.empty_cache()
    return block



def main():
    args = parse_args()
    if args.workload == "tp":
        return run_tp_arm(args)
    if args.workload == "admission":
        return run_admission_arm(args)
    if args.workload == "glue":
        return run_glue_arm(args)
    if args.workload == "backbone" and args.impl in ("b200", "reference-gpu"):
        return run_backbone_arm(args)
    if args.workload == "backbone5":
        return run_backbone5_arm(args)
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.impl == "reference-gpu":
        run_reference_gpu_arm(args)
    elif args.workload != "decode":
        run_prefill_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
