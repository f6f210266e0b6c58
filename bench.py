#!/usr/bin/env python
"""Benchmark of the GGUF quantised matrix-vector hot path on B200.

Workload (N = 1 and, as independent replicas, every N): the Llama-style 8B decode layer at
batch 1 -- q/o 4096x4096, k/v 1024x4096, gate/up 14336x4096 in Q4_K and down 4096x14336 in
Q6_K, fp32 N(0, 0.02) weights quantised by the library's own (reference-exact) quantisers,
fp32 N(0, 1) activations. A step is one pass of the seven projections over one layer; the
steps walk a stack of distinct layers, so a step's weights (138 MB, more than the 126 MB L2)
were last touched a whole stack (>1 GB) ago.

Metric: quant matvec GB/s = algorithmic bytes (weights + fp32 activations in + fp32 outputs out)
per second, whole job; ms_per_step is the time of one decode layer.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--act int8|float]

One JSON line on stdout (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402

Q4_0, Q8_0, Q4_K, Q6_K = 2, 8, 12, 14
GEOM = {Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210)}
# name, type, rows, cols, shares the activation column of the previous projection
LAYER = [
    ("q", Q4_K, 4096, 4096, False),
    ("k", Q4_K, 1024, 4096, True),
    ("v", Q4_K, 1024, 4096, True),
    ("o", Q4_K, 4096, 4096, False),
    ("gate", Q4_K, 14336, 4096, False),
    ("up", Q4_K, 14336, 4096, True),
    ("down", Q6_K, 4096, 14336, False),
]
METRIC, UNIT = "quant_matvec_GBps", "GB/s"


def algo_bytes(t: int, rows: int, cols: int, tokens: int = 1) -> int:
    per, stride = GEOM[t]
    return rows * (cols // per) * stride + 4 * cols * tokens + 4 * rows * tokens


LAYER_BYTES = sum(algo_bytes(t, r, c) for _, t, r, c, _ in LAYER)  # 138,149,888


def measured_peak_gbs():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            f = [c.strip() for c in line.split(",")]
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
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# --------------------------------------------------------------------------- CPU arm


def cpu_layer_sample(oracle, ol, blocks, xs, mode, step, threads):
    """One decode layer (seven matvecs) through the CPU oracle; returns seconds."""
    t0 = time.perf_counter()
    for (name, t, rows, cols, _), b in zip(LAYER, blocks):
        oracle.matvec(t, b, rows, cols, xs[cols], mode, step, threads=threads)
    return time.perf_counter() - t0


def host_layer_blocks(oracle, ol, seed=1):
    """The layer's weights from the oracle's counter-based generator and quantisers (host only)."""
    out = []
    for i, (name, t, rows, cols, _) in enumerate(LAYER):
        out.append(oracle.quantize(t, oracle.normal(seed, i, rows * cols, 0.02)))
    return out


def run_reference(args):
    """The reference's CPU path for this metric: the C restatement (oracle/) on every host core.
    The reference itself cannot be built here (no rustc/cargo, and it needs clang at run time)."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from tests import oracle_lib as ol

    oracle = ol.load()
    threads = os.cpu_count() or 1
    mode, step = (ol.INT8, 32) if args.act == "int8" else (ol.FLOAT_RUN, 32)
    blocks = host_layer_blocks(oracle, ol)
    xs = {4096: oracle.normal(1, 100, 4096, 1.0), 14336: oracle.normal(1, 101, 14336, 1.0)}
    for _ in range(max(args.warmup, 1)):
        cpu_layer_sample(oracle, ol, blocks, xs, mode, step, threads)
    times = [cpu_layer_sample(oracle, ol, blocks, xs, mode, step, threads) for _ in range(args.steps)]
    total = sum(times)
    value = LAYER_BYTES * args.steps / total / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 x q4/q6 -> i32, fp32 accumulate" if args.act == "int8" else "fp32",
        "data": "synthetic", "config": workload_config(args, 1, cpu=True),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{args.steps} decode layers (7 matvecs, {LAYER_BYTES} algorithmic bytes each) after {max(args.warmup, 1)} warm-up"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def workload_config(args, layers, cpu=False):
    l2 = "inputs larger than L2: each step reads a different layer of a stack larger than 1 GB"
    timing = "the K timed steps are one CUDA graph, replayed once untimed (its first launch uploads it) after the W warm-up steps, then timed with CUDA events"
    if cpu:
        l2 = "one layer (138 MB of blocks) re-read every step: larger than the host's last-level cache"
        timing = "host wall clock around the K steps, after the W warm-up steps; all host threads"
    return {"workload": "llama-8B-shaped decode layer, batch 1: q/o 4096x4096, k/v 1024x4096, gate/up 14336x4096 Q4_K; down 4096x14336 Q6_K",
            "activation_mode": "int8 records, step 32 (recipe default profile)" if args.act == "int8" else "fp32 activations as they are",
            "layers_in_rotation": layers, "l2": l2, "timing": timing,
            "algorithmic_bytes_per_step": LAYER_BYTES, "multi_gpu": "replicas only (the decode layer is unsharded)"}


# --------------------------------------------------------------------------- GPU arm


def build_layers(ctx, rq, torch, n_layers, seed, device):
    """n_layers decode layers: fp32 N(0, 0.02) on the device, quantised by the library."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    layers, first_blocks = [], []
    for li in range(n_layers):
        ws = []
        for (name, t, rows, cols, _) in LAYER:
            w32 = torch.randn(rows * cols, generator=gen, device=device, dtype=torch.float32) * 0.02
            blocks = ctx.quantize(t, w32)
            ws.append(ctx.weight_from_device(t, blocks, rows, cols))
            if li == 0:
                first_blocks.append(blocks.cpu().numpy())
            del w32, blocks
        layers.append(ws)
    torch.cuda.synchronize()
    return layers, first_blocks


def run_ours(args):
    import torch

    import recipe_dev_b200 as rq

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    ctx = rq.Context(local)
    mode = rq.ACT_INT8 if args.act == "int8" else rq.ACT_FLOAT
    cached = 2 if mode == rq.ACT_INT8 else rq.ACT_FLOAT
    step = 32
    n_layers = args.layers
    layers, first_blocks = build_layers(ctx, rq, torch, n_layers, 1 + rank, device)
    gen = torch.Generator(device=device)
    gen.manual_seed(100 + rank)
    xs = {4096: torch.randn(4096, generator=gen, device=device), 14336: torch.randn(14336, generator=gen, device=device)}
    ys = {name: torch.empty(rows, device=device) for name, _, rows, _, _ in LAYER}
    # q/k/v read one activation column, gate/up another: one call (and one launch) per group
    GROUPS = [[0, 1, 2], [3], [4, 5], [6]]

    def layer_pass(li):
        ws = layers[li % n_layers]
        for g in GROUPS:
            cols = LAYER[g[0]][3]
            ctx.matvec_multi([ws[j] for j in g], xs[cols], [ys[LAYER[j][0]] for j in g], act_mode=mode, step=step)

    # kernels of the library per step: one streaming matvec per group; an int8 group wider than 8192 inputs
    # also launches the activation quantiser (narrower ones quantise inside the matvec launch)
    launches_per_step = sum(2 if (mode == rq.ACT_INT8 and LAYER[g[0]][3] > 8192) else 1 for g in GROUPS)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # one CUDA graph per layer of the stack: a step is one graph launch, so the host's launch rate
    # does not bound the 5-20 us kernels
    for i in range(3):
        layer_pass(i)  # grows the library's scratch before capture
    torch.cuda.synchronize()
    # the W warm-up steps and the K timed steps are one CUDA graph each (as a decoder captures its whole
    # stack of layers): step i runs layer i of the rotation
    def capture(first, count):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(count):
                layer_pass(first + i)
        return g

    warm_graph = capture(0, args.warmup)
    timed_graph = capture(args.warmup, args.steps)
    stream = torch.cuda.current_stream()

    # ---- device-resident timing: exactly K steps after W warm-up steps -----------------
    warm_graph.replay()
    timed_graph.replay()  # untimed: the first launch of a graph also uploads it to the device
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    timed_graph.replay()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    ctx.check()

    # ---- dominant kernel alone: the streaming Q4_K matvec over gate+up (28672 x 4096), launches back to back
    n_dom = max(args.steps, 20)
    if mode == rq.ACT_INT8:
        ctx.matvec(layers[0][4], xs[4096], ys["gate"], act_mode=mode, step=step)  # leaves the records the cached launches read
    torch.cuda.synchronize()
    dom_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(dom_graph):
        for i in range(n_dom):
            li = i % n_layers
            ctx.matvec_multi([layers[li][4], layers[li][5]], xs[4096], [ys["gate"], ys["up"]], act_mode=mode, step=step)
    dom_graph.replay()
    torch.cuda.synchronize()
    d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    d0.record(stream)
    dom_graph.replay()
    d1.record(stream)
    torch.cuda.synchronize()
    dom_us = 1e3 * d0.elapsed_time(d1) / n_dom

    # ---- end to end: host buffers through rq_matvec_host, copies inside the timed region ----
    hx = {c: np.ascontiguousarray(v.cpu().numpy()) for c, v in xs.items()}
    def layer_pass_host(li):
        ws = layers[li % n_layers]
        out = None
        for g in GROUPS:  # one host call per group of projections that read the same x
            out = ctx.matvec_multi_host([ws[j] for j in g], hx[LAYER[g[0]][3]], act_mode=mode, step=step)
        return out
    for i in range(min(args.warmup, 3)):
        layer_pass_host(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        layer_pass_host(args.warmup + i)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    for ws in layers:
        for w in ws:
            w.free()
    sharded_out = run_sharded_configs(ctx, rq, torch, dist, rank, world, device, args.steps) if args.sharded else None
    other_out = run_other_configs(ctx, rq, torch, device) if (args.sharded and rank == 0) else None

    # max over ranks
    if dist is not None:
        t = torch.tensor([ms, e2e_s], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1])
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    total_bytes = LAYER_BYTES * args.steps * world
    value = total_bytes / (ms * 1e-3) / 1e9
    peak, peak_kind = measured_peak_gbs()
    dom_bytes = 2 * algo_bytes(Q4_K, 14336, 4096) - 4 * 4096  # two row sets, one activation column
    achieved = dom_bytes / (dom_us * 1e-6) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 x q4/q6 -> i32, fp32 accumulate" if mode == rq.ACT_INT8 else "fp32",
        "data": "synthetic", "config": workload_config(args, n_layers),
        "us_per_decode_layer": 1e3 * ms / args.steps,
        "frac_of_hbm_measured": value / world / peak, "frac_of_hbm_nominal_8TBs": value / world / 8000.0,
        "roofline": {"bound": "hbm", "kernel": "rq_gemv_stream_kernel<Q4_K> over gate+up (2 x 14336 x 4096), one launch", "achieved": achieved, "peak": peak,
                     "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})", "unit": "GB/s", "frac": achieved / peak,
                     "us_per_launch": dom_us, "algorithmic_bytes_per_launch": dom_bytes,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the same kernel over one of the two
                     # row sets (14336 x 4096: 33.11 MB read, nothing written), scaled to the launch's two row sets
                     "traffic": 2 * 33_106_400, "traffic_source": "profiles/rq_gemv_stream_q4k_14336x4096_int8.md, x2 row sets"},
        "e2e": {"value": total_bytes / e2e_s / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": sum(4 * c for _, _, _, c, _ in LAYER), "d2h_bytes_per_step": sum(4 * r for _, _, r, _, _ in LAYER),
                "ms_per_step": 1e3 * e2e_s / args.steps, "call": "rq_matvec_multi_host x 4 per step (q/k/v, o, gate/up, down: host x in, host y out)"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    if sharded_out is not None:
        line["sharded"] = sharded_out
    if other_out is not None:
        line["other_configs"] = other_out
    if args.cpu_baseline:
        from tests import oracle_lib as ol

        oracle = ol.load()
        threads = os.cpu_count() or 1
        omode = ol.INT8 if mode == rq.ACT_INT8 else ol.FLOAT_RUN
        t0 = time.perf_counter()
        reps = 0
        while reps < 1 or (time.perf_counter() - t0 < 10.0 and reps < 50):
            cpu_layer_sample(oracle, ol, first_blocks, hx, omode, step, threads)
            reps += 1
        cpu_s = (time.perf_counter() - t0) / reps
        line["cpu_baseline"] = {"value": LAYER_BYTES / cpu_s / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
                                "ms_per_step": 1e3 * cpu_s,
                                "sample": f"{reps} passes of one decode layer (layer 0 of the stack, same blocks and activations) through oracle/rq_oracle.c"}
    emit(line)
    if dist is not None:
        dist.destroy_process_group()


def run_case(args):
    """A small single-kernel case for profiling: `--case q4k:14336x4096:int8[:tokens]` runs the
    matvec of that shape over `--layers` distinct weight copies (so launches do not hit L2) for
    `--steps` launches after `--warmup`, and prints the mean time per launch."""
    import torch

    import recipe_dev_b200 as rq

    parts = args.case.split(":")
    t = {"q4k": rq.Q4_K, "q6k": rq.Q6_K, "q8_0": rq.Q8_0, "q4_0": rq.Q4_0}[parts[0]]
    rows, cols = (int(v) for v in parts[1].split("x"))
    mode = rq.ACT_INT8 if parts[2] == "int8" else rq.ACT_FLOAT
    tokens = int(parts[3]) if len(parts) > 3 else 1
    torch.cuda.set_device(0)
    ctx = rq.Context(0)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4)
    ws = []
    for _ in range(args.layers):
        w32 = torch.randn(rows * cols, generator=gen, device="cuda") * 0.02
        ws.append(ctx.weight_from_device(t, ctx.quantize(t, w32), rows, cols))
        del w32
    x = torch.randn(tokens, cols, generator=gen, device="cuda")
    y = torch.empty(tokens, rows, device="cuda")
    stream = torch.cuda.current_stream()
    cached = 2 if mode == rq.ACT_INT8 else mode
    if args.matmul:
        # the batched entry point: time per call (the activation split and, for split K, the sum kernel included)
        for i in range(args.warmup):
            ctx.matmul(ws[i % len(ws)], x, y, act_mode=mode, step=32, stream=stream)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(args.steps):
            ctx.matmul(ws[(args.warmup + i) % len(ws)], x, y, act_mode=mode, step=32, stream=stream)
        e1.record(stream)
        torch.cuda.synchronize()
        us = 1e3 * e0.elapsed_time(e1) / args.steps
        flops = 2.0 * rows * cols * tokens
        emit({"case": args.case, "entry": "rq_matmul", "us_per_call": us, "TFLOPs_useful": flops / us / 1e6, "TFLOPs_issued_fp16": 3 * flops / us / 1e6,
                          "calls": args.steps, "weight_copies": args.layers})
        ctx.check()
        return
    ctx.matvec(ws[0], x, y, act_mode=mode, step=32, stream=stream)
    for i in range(args.warmup):
        ctx.matvec(ws[i % len(ws)], x, y, act_mode=cached, step=32, stream=stream)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.graph:
        # the launches as one CUDA graph, so that the host's launch rate does not bound short kernels
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(args.steps):
                ctx.matvec(ws[(args.warmup + i) % len(ws)], x, y, act_mode=cached, step=32)
        g.replay()
        torch.cuda.synchronize()
        e0.record()
        g.replay()
        e1.record()
    else:
        e0.record(stream)
        for i in range(args.steps):
            ctx.matvec(ws[(args.warmup + i) % len(ws)], x, y, act_mode=cached, step=32, stream=stream)
        e1.record(stream)
    torch.cuda.synchronize()
    us = 1e3 * e0.elapsed_time(e1) / args.steps
    per, stride = {rq.Q4_K: (256, 144), rq.Q6_K: (256, 210), rq.Q8_0: (32, 34), rq.Q4_0: (32, 18)}[t]
    nbytes = rows * (cols // per) * stride + 4 * cols * tokens + 4 * rows * tokens
    peak, kind = measured_peak_gbs()
    emit({"case": args.case, "us_per_launch": us, "GBps": nbytes / us / 1e3, "frac_of_hbm": nbytes / us / 1e3 / peak,
                      "peak": f"{peak} ({kind})", "algorithmic_bytes": nbytes, "launches": args.steps, "weight_copies": args.layers, "graph": bool(args.graph)})


def run_sharded_configs(ctx, rq, torch, dist, rank, world, device, steps):
    """The two configs that shard across GPUs, timed on the device (max over ranks):
    the row-split Q6_K LM head (262144 x 2560, logits all-gathered) at batch 1 and 4, and the
    expert-parallel Q4_K MoE bank (256 experts, top-8, hidden 2048, ffn 512, gated shared expert on
    rank 0, outputs all-reduced) at batch 1 and 16. Returns a dict for the JSON line."""
    from recipe_dev_b200 import sharded

    out = {}
    stream = torch.cuda.current_stream()

    def timed(fn, reps):
        """Mean device time of fn, max over ranks. The reps are captured into one CUDA graph (kernels and the NCCL
        collective alike), so the host's launch rate is not what is measured; if capture is refused the reps run eagerly."""
        for _ in range(3):
            fn()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        graph = None
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(reps):
                    fn()
            g.replay()  # the first launch uploads the graph
            torch.cuda.synchronize()
            graph = g
        except Exception as exc:  # noqa: BLE001 - any capture failure falls back to eager timing
            print(f"bench.py: graph capture of a sharded step failed ({type(exc).__name__}: {exc}); timing eager launches", file=sys.stderr)
            torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        if graph is not None:
            graph.replay()
        else:
            for _ in range(reps):
                fn()
        e1.record(stream)
        torch.cuda.synchronize()
        us = torch.tensor([1e3 * e0.elapsed_time(e1) / reps], device=device, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(us, op=dist.ReduceOp.MAX)
        timed.graphed = graph is not None
        return float(us[0])

    # ---- LM head: rows [first, first + count) of 262144 x 2560 Q6_K on this rank
    rows, cols = 262144, 2560
    first, count = sharded.shard_range(rows, world, rank)
    gen = torch.Generator(device=device)
    gen.manual_seed(2000 + rank)
    copies = []
    for _ in range(2 if count * cols // 256 * 210 < 200_000_000 else 1):  # small shares rotate two copies so L2 cannot hold them
        w32 = torch.randn(count * cols, generator=gen, device=device) * 0.02
        copies.append(ctx.weight_from_device(Q6_K, ctx.quantize(Q6_K, w32), count, cols))
        del w32
    mode = rq.ACT_INT8
    for tokens in (1, 4):
        x = torch.randn(tokens, cols, generator=gen, device=device)
        local = torch.empty(tokens, count, device=device)
        it = [0]

        def head_step():
            ctx.matvec(copies[it[0] % len(copies)], x, local, act_mode=mode, step=32)
            it[0] += 1
            return sharded.gather_rows(local, rows, dist, world, rank)

        us = timed(head_step, max(10, steps // 10))
        nbytes = rows * (cols // 256) * 210 + 4 * cols * tokens + 4 * rows * tokens
        out[f"lm_head_q6k_262144x2560_batch{tokens}"] = {"us": us, "GBps": nbytes / us / 1e3, "algorithmic_bytes": nbytes,
                                                         "rows_per_gpu": count, "collective": "all_gather fp32 logits" if world > 1 else "none",
                                                         "launch": "cuda graph" if timed.graphed else "eager"}
    for w in copies:
        w.free()
    del copies
    # ---- MoE bank: experts [first, first + count) of 256 on this rank
    experts, top, hidden, ffn = 256, 8, 2048, 512
    ef, ec = sharded.shard_range(experts, world, rank)
    gen.manual_seed(3000 + rank)

    def host_blocks(n_rows, n_cols):
        w32 = torch.randn(n_rows * n_cols, generator=gen, device=device) * 0.02
        b = ctx.quantize(Q4_K, w32).cpu().numpy()
        del w32
        return b

    gate, up, down = host_blocks(ec * ffn, hidden), host_blocks(ec * ffn, hidden), host_blocks(ec * hidden, ffn)
    shared = None
    if rank == 0:
        shared = (host_blocks(ffn, hidden), host_blocks(ffn, hidden), host_blocks(hidden, ffn), (torch.randn(hidden, generator=gen, device=device) * 0.02).cpu().numpy())
    bank = ctx.moe_prepare(Q4_K, gate, up, down, ec, hidden, ffn, shared=shared)
    del gate, up, down
    rgen = torch.Generator(device=device)
    rgen.manual_seed(3999)  # the router scores are the same on every rank (the router is replicated)
    expert_bytes = 3 * ffn * (hidden // 256) * 144
    for tokens in (1, 16):
        scores = torch.randn(experts, tokens, generator=rgen, device=device)
        xm = torch.randn(hidden, tokens, generator=rgen, device=device)
        y = torch.empty(hidden, tokens, device=device)

        def moe_step():
            routing = ctx.moe_route(scores, top)
            ctx.moe_forward(bank, xm, routing, top, include_shared=(rank == 0), y=y)  # the whole routing plane: a rank reads its experts' rows
            if dist is not None:
                dist.all_reduce(y)
            return y

        us = timed(moe_step, max(10, steps // 10))
        nbytes = tokens * ((top + 1) * expert_bytes + (top + 1) * 3 * 4 * (hidden + ffn))
        loads = sharded.routed_bytes_per_rank(ctx.moe_route(scores, top), experts, world, expert_bytes)
        out[f"moe_q4k_256e_top8_batch{tokens}"] = {"us": us, "GBps": nbytes / us / 1e3, "algorithmic_bytes": nbytes, "experts_per_gpu": ec,
                                                  "routed_bytes_per_rank_min_max": [min(loads), max(loads)],
                                                  "collective": "all_reduce fp32 [hidden, tokens]" if world > 1 else "none",
                                                  "launch": "cuda graph" if timed.graphed else "eager"}
    ctx.check()
    bank.free()
    return out


def run_other_configs(ctx, rq, torch, device):
    """BASELINE's remaining single-GPU configs, device-timed on rank 0 (not the headline: recorded beside it):
    the Q8_0 4096 x 4096 matvec (int8, one token) and the batched tensor-core product at 16 / 64 / 512 tokens."""
    out = {}
    gen = torch.Generator(device=device)
    gen.manual_seed(5)
    stream = torch.cuda.current_stream()

    def quantised(t, rows, cols, copies):
        ws = []
        for _ in range(copies):
            w32 = torch.randn(rows * cols, generator=gen, device=device) * 0.02
            ws.append(ctx.weight_from_device(t, ctx.quantize(t, w32), rows, cols))
            del w32
        return ws

    def graph_time(fn, reps):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(reps):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        g.replay()
        e1.record(stream)
        torch.cuda.synchronize()
        return 1e3 * e0.elapsed_time(e1) / reps

    # cfg 1: Q8_0 4096 x 4096, eight copies in rotation (143 MB: larger than L2)
    ws = quantised(Q8_0, 4096, 4096, 8)
    x = torch.randn(4096, generator=gen, device=device)
    y = torch.empty(4096, device=device)
    us = graph_time(lambda i: ctx.matvec(ws[i % 8], x, y, act_mode=rq.ACT_INT8, step=32), 64)
    nbytes = algo_bytes(Q8_0, 4096, 4096)
    out["q8_0_4096x4096_int8_batch1"] = {"us": us, "GBps": nbytes / us / 1e3, "algorithmic_bytes": nbytes}
    for w in ws:
        w.free()
    # cfg 5: the batched product, fp32 activations, tensor cores
    for name, t, rows, cols in (("q4k_14336x4096", Q4_K, 14336, 4096), ("q6k_4096x14336", Q6_K, 4096, 14336)):
        ws = quantised(t, rows, cols, 4)
        for tokens in (16, 64, 512):
            xb = torch.randn(tokens, cols, generator=gen, device=device)
            yb = torch.empty(tokens, rows, device=device)
            for i in range(2):
                ctx.matmul(ws[i], xb, yb)  # grows the scratch before timing
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(8):
                ctx.matmul(ws[i % 4], xb, yb)
            e1.record(stream)
            torch.cuda.synchronize()
            us = 1e3 * e0.elapsed_time(e1) / 8
            out[f"matmul_{name}_tokens{tokens}"] = {"us": us, "TFLOPs_useful": 2.0 * rows * cols * tokens / us / 1e6}
        for w in ws:
            w.free()
    ctx.check()
    return out


RESULT_OUT = None


def emit(line):
    """The run's one JSON line, on the process's original standard output."""
    out = RESULT_OUT or sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    # Standard output carries the JSON line and nothing else: libraries that write to file descriptor 1 on their
    # own (NCCL prints its version there) are sent to standard error for the whole run.
    global RESULT_OUT
    sys.stdout.flush()
    RESULT_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default=None, help="profile one matvec shape, e.g. q4k:14336x4096:int8")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--act", default="int8", choices=["int8", "float"])
    ap.add_argument("--layers", type=int, default=8, help="distinct decode layers in rotation (138 MB each)")
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false")
    ap.add_argument("--no-sharded", dest="sharded", action="store_false", help="skip the row-split LM head and expert-parallel MoE configs")
    ap.add_argument("--graph", action="store_true", help="--case: replay the launches as one CUDA graph")
    ap.add_argument("--matmul", action="store_true", help="--case: the batched tensor-core entry point (rq_matmul) instead of rq_matvec")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
