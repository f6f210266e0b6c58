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
GEOM = {Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210), 3: (32, 20)}  # 3 = Q4_1, the storage of int4 sums
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


# --------------------------------------------------------------------------- shared inputs


def oracle_normal(oracle, seed: int, stream: int, count: int, sigma: float) -> np.ndarray:
    """`count` values of the oracle's counter-based generator (value i depends on (seed, stream, i) only), drawn in
    parallel chunks: the same numbers as one call, in a fraction of the time."""
    import concurrent.futures

    out = np.empty(count, dtype=np.float32)
    chunk = 1 << 22
    spans = [(first, min(chunk, count - first)) for first in range(0, count, chunk)]

    def fill(span):
        first, n = span
        out[first:first + n] = oracle.normal(seed, stream, n, sigma, first=first)

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as pool:
        list(pool.map(fill, spans))
    return out


LAYER_SEED = 1  # BASELINE: the decode layer's weights are seed 1, one sub-stream per tensor in the order q, k, v, o, gate, up, down


def layer_inputs(oracle):
    """The activations both arms read: fp32 N(0, 1), seed 1, sub-streams 100 (4096 inputs) and 101 (14336 inputs)."""
    return {4096: oracle.normal(LAYER_SEED, 100, 4096, 1.0), 14336: oracle.normal(LAYER_SEED, 101, 14336, 1.0)}


# --------------------------------------------------------------------------- CPU arm


def cpu_layer_sample(oracle, ol, blocks, xs, mode, step, threads):
    """One decode layer (seven matvecs) through the CPU oracle; returns seconds."""
    t0 = time.perf_counter()
    for (name, t, rows, cols, _), b in zip(LAYER, blocks):
        oracle.matvec(t, b, rows, cols, xs[cols], mode, step, threads=threads)
    return time.perf_counter() - t0


def host_layer_blocks(oracle, ol, seed=LAYER_SEED):
    """The layer's weights from the oracle's counter-based generator and quantisers (host only)."""
    out = []
    for i, (name, t, rows, cols, _) in enumerate(LAYER):
        out.append(oracle.quantize(t, oracle_normal(oracle, seed, i, rows * cols, 0.02)))
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
    xs = layer_inputs(oracle)
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
    timing = ("the K timed steps are one CUDA graph, replayed once untimed (its first launch uploads it) after the W warm-up steps, then timed with "
              "CUDA events; the graph is then replayed 20 more times for the spread (repeat_ms)")
    if cpu:
        l2 = "one layer (138 MB of blocks) re-read every step: larger than the host's last-level cache"
        timing = "host wall clock around the K steps, after the W warm-up steps; all host threads"
    return {"workload": "llama-8B-shaped decode layer, batch 1: q/o 4096x4096, k/v 1024x4096, gate/up 14336x4096 Q4_K; down 4096x14336 Q6_K",
            "activation_mode": "int8 records, step 32 (recipe default profile)" if args.act == "int8" else "fp32 activations as they are",
            "seeds": "weights seed 1, one sub-stream per tensor (q, k, v, o, gate, up, down); activations seed 1, sub-streams 100 / 101; the oracle's counter-based generator",
            "layers_in_rotation": layers, "l2": l2, "timing": timing,
            "algorithmic_bytes_per_step": LAYER_BYTES, "multi_gpu": "replicas only (the decode layer is unsharded)"}


# --------------------------------------------------------------------------- GPU arm


def rel_err(y, ref) -> float:
    """max_i |y_i - ref_i| / max(|ref_i|, 1e-3 max|ref|): the error measure of the parity tests."""
    y, ref = np.asarray(y, np.float64), np.asarray(ref, np.float64)
    floor = 1e-3 * np.max(np.abs(ref))
    return float(np.max(np.abs(y - ref) / np.maximum(np.abs(ref), floor)))


def build_layers(ctx, rq, torch, oracle, n_layers, rank, device):
    """n_layers decode layers on the device. Layer 0 is BASELINE's: fp32 N(0, 0.02) from the oracle's generator at seed 1
    (the CPU arm's weights), quantised on the device (byte-exact with the oracle's quantisers); the other layers of the
    rotation exist only so that a step's weights are cold, and come from the device's own generator."""
    gen = torch.Generator(device=device)
    gen.manual_seed(1000 + rank)
    layers, first_blocks = [], []
    for li in range(n_layers):
        ws = []
        for i, (name, t, rows, cols, _) in enumerate(LAYER):
            if li == 0:
                w32 = torch.from_numpy(oracle_normal(oracle, LAYER_SEED, i, rows * cols, 0.02)).to(device)
            else:
                w32 = torch.randn(rows * cols, generator=gen, device=device, dtype=torch.float32) * 0.02
            blocks = ctx.quantize(t, w32)
            ws.append(ctx.weight_from_device(t, blocks, rows, cols))
            if li == 0:
                first_blocks.append(blocks.cpu().numpy())
            del w32, blocks
        layers.append(ws)
    torch.cuda.synchronize()
    return layers, first_blocks


def profile_traffic(name: str):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch from a committed ncu summary (its `dram_bytes_per_launch:` line)."""
    path = ROOT / "profiles" / name
    try:
        for line in path.read_text().splitlines():
            if line.startswith("dram_bytes_per_launch:"):
                return int(line.split(":")[1].split()[0].replace(",", ""))
    except OSError:
        pass
    return None


def run_ours(args):
    import torch

    import recipe_dev_b200 as rq
    from tests import oracle_lib as ol

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    oracle = ol.load()  # the checker and the source of BASELINE's seeded inputs; nothing timed on the GPU runs through it
    ctx = rq.Context(local)
    mode = rq.ACT_INT8 if args.act == "int8" else rq.ACT_FLOAT
    step = 32
    n_layers = args.layers
    layers, first_blocks = build_layers(ctx, rq, torch, oracle, n_layers, rank, device)
    hx = layer_inputs(oracle)
    xs = {4096: torch.from_numpy(hx[4096]).to(device)}
    ys = {name: torch.empty(rows, device=device) for name, _, rows, _, _ in LAYER}
    # q/k/v read one activation column, gate/up another: one call (and one launch) per group
    GROUPS = [[0, 1, 2], [3], [4, 5], [6]]
    ctx.reserve(14336, 14336, 1)  # no call below grows a work area: nothing allocates or synchronises inside a timed region

    # The layer's launches are chained: o reads q's output plane (attention itself is not on this path), gate / up read
    # o's, down reads gate's; the planes between the launches never leave the device.
    SOURCE = {0: None, 3: "q", 4: "o", 6: "gate"}

    def layer_pass(li, stream=None):
        ws = layers[li % n_layers]
        for g in GROUPS:
            src = SOURCE[g[0]]
            x_in = xs[4096] if src is None else ys[src]
            ctx.matvec_multi([ws[j] for j in g], x_in, [ys[LAYER[j][0]] for j in g], act_mode=mode, step=step, stream=stream)

    # kernels of the library per step: one streaming matvec per group; an int8 group wider than 8192 inputs
    # also launches the activation quantiser (narrower ones quantise inside the matvec launch)
    launches_per_step = sum(2 if (mode == rq.ACT_INT8 and LAYER[g[0]][3] > 8192) else 1 for g in GROUPS)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(3):
        layer_pass(i)  # module load before capture
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
    # the spread: the same K steps twenty more times, each timed on its own
    repeats = []
    for _ in range(20):
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record(stream)
        timed_graph.replay()
        r1.record(stream)
        torch.cuda.synchronize()
        repeats.append(r0.elapsed_time(r1))
    ctx.check()

    # ---- what the timed kernels computed, against the oracle: layer 0 (BASELINE's seeded layer), a sample of rows of each projection
    layer_pass(0)
    torch.cuda.synchronize()
    omode = ol.INT8 if mode == rq.ACT_INT8 else ol.FLOAT_RUN
    worst = 0.0
    rng = np.random.default_rng(7)
    host_planes = {name: ys[name].cpu().numpy() for name in ys}
    reads = {"q": None, "k": None, "v": None, "o": "q", "gate": "o", "up": "o", "down": "gate"}
    for (name, t, rows, cols, _), blocks in zip(LAYER, first_blocks):
        pick = np.sort(rng.choice(rows, size=32, replace=False))
        row_bytes = cols // GEOM[t][0] * GEOM[t][1]
        sub = blocks.reshape(rows, row_bytes)[pick].reshape(-1)
        x_in = hx[4096] if reads[name] is None else host_planes[reads[name]]  # each projection against the input it really read
        ref = oracle.matvec(t, sub, pick.size, cols, x_in, omode, step)
        worst = max(worst, rel_err(host_planes[name][pick], ref))
    if worst > 1e-3:
        raise SystemExit(f"bench.py: the timed kernels' outputs differ from the CPU oracle by {worst:.3e} (bar 1e-3)")

    # ---- dominant kernel alone: the streaming Q4_K matvec over gate+up (28672 x 4096), launches back to back
    n_dom = max(args.steps, 20)
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

    # ---- end to end: one boundary crossing per step. Each layer of the rotation is a recorded sequence of its four calls;
    # a step copies x in from host memory, replays the sequence, copies the step's result (down's output) back, synchronises.
    sequences = []
    for li in range(n_layers):
        s = ctx.sequence_begin()
        layer_pass(li, stream=s)
        sequences.append(ctx.sequence_end())
    host_out = np.empty(4096, np.float32)
    for i in range(max(args.warmup, 3)):
        sequences[i % n_layers].run_host(hx[4096], xs[4096], ys["down"], host_out)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        sequences[(args.warmup + i) % n_layers].run_host(hx[4096], xs[4096], ys["down"], host_out)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_err = rel_err(host_out, ys["down"].cpu().numpy())
    clocks = sampler.stop() if rank == 0 else None
    for sq in sequences:
        sq.free()
    for ws in layers:
        for w in ws:
            w.free()
    sharded_out = run_sharded_configs(ctx, rq, torch, dist, rank, world, device, args.steps) if args.sharded else None
    other_out = run_other_configs(ctx, rq, torch, oracle, ol, device) if (args.sharded and rank == 0) else None

    # max over ranks
    if dist is not None:
        t = torch.tensor([ms, e2e_s, worst], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s, worst = float(t[0]), float(t[1]), float(t[2])
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    total_bytes = LAYER_BYTES * args.steps * world
    value = total_bytes / (ms * 1e-3) / 1e9
    peak, peak_kind = measured_peak_gbs()
    dom_bytes = 2 * algo_bytes(Q4_K, 14336, 4096) - 4 * 4096  # two row sets, one activation column
    achieved = dom_bytes / (dom_us * 1e-6) / 1e9
    one_set = profile_traffic("rq_gemv_stream_q4k_14336x4096_int8.md")
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 x q4/q6 -> i32, fp32 accumulate" if mode == rq.ACT_INT8 else "fp32",
        "data": "synthetic", "config": workload_config(args, n_layers),
        "us_per_decode_layer": 1e3 * ms / args.steps,
        "repeat_ms": {"n": len(repeats), "median": statistics.median(repeats), "p99": sorted(repeats)[-1], "min": min(repeats)},
        "max_rel_err_vs_oracle": worst,
        "frac_of_hbm_measured": value / world / peak, "frac_of_hbm_nominal_8TBs": value / world / 8000.0,
        "roofline": {"bound": "hbm", "kernel": "rq_gemv_stream_kernel<Q4_K> over gate+up (2 x 14336 x 4096), one launch", "achieved": achieved, "peak": peak,
                     "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})", "unit": "GB/s", "frac": achieved / peak,
                     "us_per_launch": dom_us, "algorithmic_bytes_per_launch": dom_bytes,
                     # an ncu capture of the same kernel over one of the two row sets (14336 x 4096), scaled to the launch's two:
                     # traffic grows with the rows read
                     "traffic": None if one_set is None else 2 * one_set,
                     "traffic_source": "profiles/rq_gemv_stream_q4k_14336x4096_int8.md (dram_bytes_per_launch), x2 row sets"},
        "e2e": {"value": total_bytes / e2e_s / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": 4 * 4096, "d2h_bytes_per_step": 4 * 4096,
                "ms_per_step": 1e3 * e2e_s / args.steps, "result_equals_device_plane": e2e_err == 0.0,
                "call": "rq_sequence_run_host: x copied in from host memory, the layer's four recorded calls replayed as one submission "
                        "(o reads q's plane, gate/up read o's, down reads gate's: the planes between stay on the device), down's output copied "
                        "back, one synchronisation"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    if sharded_out is not None:
        line["sharded"] = sharded_out
    if other_out is not None:
        line["other_configs"] = other_out
    if args.cpu_baseline:
        threads = os.cpu_count() or 1
        t0 = time.perf_counter()
        reps = 0
        while reps < 1 or (time.perf_counter() - t0 < 10.0 and reps < 50):
            cpu_layer_sample(oracle, ol, first_blocks, hx, omode, step, threads)  # the CPU arm's fixed inputs: the same bytes and flops
            reps += 1
        cpu_s = (time.perf_counter() - t0) / reps
        line["cpu_baseline"] = {"value": LAYER_BYTES / cpu_s / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
                                "ms_per_step": 1e3 * cpu_s,
                                "sample": f"{reps} passes of one decode layer (BASELINE's seeded layer: the same blocks and activations the GPU arm timed as layer 0) through oracle/rq_oracle.c"}
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
        if args.graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(args.steps):
                    ctx.matmul(ws[(args.warmup + i) % len(ws)], x, y, act_mode=mode, step=32)
            g.replay()
            torch.cuda.synchronize()
            e0.record()
            g.replay()
            e1.record()
        else:
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
    """The two configs that shard across GPUs, timed on the device (max over ranks), each through the C ABI end to end:
    the row-split Q6_K LM head (262144 x 2560; the ranks' logit slices gathered) at batch 1 and 4, and the expert-parallel
    Q4_K MoE bank (256 experts, top-8, hidden 2048, ffn 512, gated shared expert on rank 0; the ranks' outputs summed in
    rank order) at batch 1 and 16. The exchange is the library's own kernel over NVLink peer memory (rq_exchange_*); the
    same step through NCCL (rq_allgather_rows / rq_allreduce_sum) is timed beside it. After timing, outside every timed
    region, rank 0 recomputes the whole config on its one GPU and the exchanged result is compared with it."""
    from recipe_dev_b200 import sharded

    out = {}
    stream = torch.cuda.current_stream()
    gloo = dist.new_group(backend="gloo") if dist is not None else None  # the host-side channel for handles and ids

    def share(obj):
        if dist is None:
            return [obj]
        got = [None] * world
        dist.all_gather_object(got, obj, group=gloo)
        return got

    def timed(fn, reps):
        """Mean device time of fn, max over ranks. The reps are captured into one CUDA graph (the library's kernels and, in
        the NCCL variant, the collective alike), so the host's launch rate is not what is measured."""
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

    nccl = None
    if world > 1:
        ids = share(rq.NcclComm.unique_id() if rank == 0 else None)
        nccl = rq.NcclComm.create(ctx, ids[0], world, rank)
    reps = max(10, steps // 10)

    # ---- LM head: rows [first, first + count) of 262144 x 2560 Q6_K on this rank. Rank r's share is drawn from the
    # device generator at seed 2000 + r, so rank 0 can draw every share again for the check.
    rows, cols = 262144, 2560
    first, count = sharded.shard_range(rows, world, rank)

    def head_share(r, n_rows):
        gen = torch.Generator(device=device)
        gen.manual_seed(2000 + r)
        w32 = torch.randn(n_rows * cols, generator=gen, device=device) * 0.02
        w = ctx.weight_from_device(Q6_K, ctx.quantize(Q6_K, w32), n_rows, cols)
        del w32
        return w

    copies = [head_share(rank, count)]
    if count * cols // 256 * 210 < 200_000_000:  # small shares rotate a second copy so L2 cannot hold them
        copies.append(head_share(100 + rank, count))
    xgen = torch.Generator(device=device)
    xgen.manual_seed(2999)  # the hidden vectors are the same on every rank (x is replicated)
    ctx.reserve(count, cols, 4)
    for tokens in (1, 4):
        x = torch.randn(tokens, cols, generator=xgen, device=device)
        local = torch.empty(tokens, count, device=device)
        gathered = torch.empty(world, tokens * count, device=device)
        ex = rq.Exchange(ctx, rank, world, tokens * count * 4)
        ex.connect(share(ex.ipc_handle()))
        it = [0]

        def compute():
            ctx.matvec(copies[it[0] % len(copies)], x, local, act_mode=rq.ACT_INT8, step=32)
            it[0] += 1

        def head_step():
            compute()
            if world > 1:
                ex.gather(local.reshape(-1), gathered)

        def head_step_nccl():
            compute()
            nccl.allgather_rows(local.reshape(-1), gathered)

        compute_us = timed(compute, reps)
        us = timed(head_step, reps) if world > 1 else compute_us
        graphed = timed.graphed
        nccl_us = timed(head_step_nccl, reps) if world > 1 else None
        # the check: the first copy's shares, gathered through the exchange, against rank 0's own product over every share
        it[0] = 0
        head_step()
        torch.cuda.synchronize()
        err = 0.0
        if world > 1 and rank == 0:
            got = gathered.view(world, tokens, count)
            for r in range(world):
                wr = copies[0] if r == 0 else head_share(r, sharded.shard_range(rows, world, r)[1])
                want = ctx.matvec(wr, x, act_mode=rq.ACT_INT8, step=32)
                err = max(err, rel_err(got[r].cpu().numpy(), want.cpu().numpy()))
                if r:
                    wr.free()
            if err > 1e-3:
                raise SystemExit(f"bench.py: gathered LM-head logits differ from a one-GPU product by {err:.3e}")
        if dist is not None:
            dist.barrier()
        nbytes = rows * (cols // 256) * 210 + 4 * cols * tokens + 4 * rows * tokens
        out[f"lm_head_q6k_262144x2560_batch{tokens}"] = {
            "us": us, "compute_us": compute_us, "exchange_us": us - compute_us, "nccl_variant_us": nccl_us, "GBps": nbytes / us / 1e3,
            "algorithmic_bytes": nbytes, "rows_per_gpu": count, "max_rel_err": err,
            "exchange": "rq_exchange_gather: peer stores over NVLink + one flag per peer, the library's own kernel" if world > 1 else "none",
            "checked": "gathered logits against rank 0's own product over every share" if world > 1 else "single GPU: nothing to gather",
            "launch": "cuda graph" if graphed else "eager"}
        ex.free()
    for w in copies:
        w.free()
    del copies

    # ---- MoE bank: experts [ef, ef + ec) of 256 on this rank. The whole bank is drawn from one seed on every rank (the
    # tensors are the model's), so that the shares belong to one bank and rank 0 can hold it whole for the check.
    experts, top, hidden, ffn = 256, 8, 2048, 512
    ef, ec = sharded.shard_range(experts, world, rank)
    bgen = torch.Generator(device=device)
    bgen.manual_seed(3000)

    def host_blocks(n_rows, n_cols):
        parts = []
        chunk_rows = max(1, (1 << 26) // n_cols)
        for r0 in range(0, n_rows, chunk_rows):
            nr = min(chunk_rows, n_rows - r0)
            w32 = torch.randn(nr * n_cols, generator=bgen, device=device) * 0.02
            parts.append(ctx.quantize(Q4_K, w32).cpu().numpy())
            del w32
        return np.concatenate(parts)

    gate, up, down = host_blocks(experts * ffn, hidden), host_blocks(experts * ffn, hidden), host_blocks(experts * hidden, ffn)
    shared = (host_blocks(ffn, hidden), host_blocks(ffn, hidden), host_blocks(hidden, ffn), (torch.randn(hidden, generator=bgen, device=device) * 0.02).cpu().numpy())
    bank = ctx.moe_prepare(Q4_K, gate, up, down, experts, hidden, ffn, expert_first=ef, expert_count=ec, shared=shared if rank == 0 else None)
    rgen = torch.Generator(device=device)
    rgen.manual_seed(3999)  # the router scores are the same on every rank (the router is replicated)
    expert_bytes = 3 * ffn * (hidden // 256) * 144
    for tokens in (1, 16):
        scores = torch.randn(experts, tokens, generator=rgen, device=device)
        xm = torch.randn(hidden, tokens, generator=rgen, device=device)
        part = torch.empty(hidden, tokens, device=device)
        y = torch.empty(hidden, tokens, device=device)
        ex = rq.Exchange(ctx, rank, world, hidden * tokens * 4)
        ex.connect(share(ex.ipc_handle()))

        weights = torch.empty_like(scores)

        def compute():
            # router scores -> routing weights -> this rank's experts, one call (routing and planning share a launch); the whole
            # routing plane is computed on every rank (the router is replicated) and a rank reads its experts' rows of it
            ctx.moe_route_forward(bank, scores, xm, top, include_shared=(rank == 0), weights=weights, y=part)
            return weights

        def moe_step():
            compute()
            if world > 1:
                ex.reduce(part.reshape(-1), y.reshape(-1))

        def moe_step_nccl():
            compute()
            nccl.allreduce_sum(part.reshape(-1), y.reshape(-1))

        compute_us = timed(compute, reps)
        us = timed(moe_step, reps) if world > 1 else compute_us
        graphed = timed.graphed
        nccl_us = timed(moe_step_nccl, reps) if world > 1 else None
        moe_step()
        torch.cuda.synchronize()
        result = (y if world > 1 else part).cpu().numpy()
        err = 0.0
        if world > 1 and rank == 0:
            whole = ctx.moe_prepare(Q4_K, gate, up, down, experts, hidden, ffn, shared=shared)
            want = ctx.moe_forward(whole, xm, ctx.moe_route(scores, top), top).cpu().numpy()
            whole.free()
            err = rel_err(result, want)
            if err > 1e-3:
                raise SystemExit(f"bench.py: the summed MoE output differs from a one-GPU bank by {err:.3e}")
        if dist is not None:
            dist.barrier()
        nbytes = tokens * ((top + 1) * expert_bytes + (top + 1) * 3 * 4 * (hidden + ffn))
        per_rank = sharded.routed_bytes_per_rank(compute(), experts, world, expert_bytes)
        torch.cuda.synchronize()
        out[f"moe_q4k_256e_top8_batch{tokens}"] = {
            "us": us, "compute_us": compute_us, "exchange_us": us - compute_us, "nccl_variant_us": nccl_us, "GBps": nbytes / us / 1e3,
            "algorithmic_bytes": nbytes, "experts_per_gpu": ec, "routed_bytes_per_rank_min_max": [min(per_rank), max(per_rank)], "max_rel_err": err,
            "exchange": "rq_exchange_reduce: peer stores over NVLink, slots added in rank order by the library's own kernel" if world > 1 else "none",
            "checked": "summed output against the whole bank on rank 0's one GPU" if world > 1 else "single GPU: nothing to sum",
            "launch": "cuda graph" if graphed else "eager"}
        ex.free()
    bank.free()
    if nccl is not None:
        nccl.destroy()
    ctx.check()
    return out


def run_other_configs(ctx, rq, torch, oracle, ol, device):
    """BASELINE's remaining single-GPU configs, device-timed on rank 0 (not the headline: recorded beside it): the Q8_0
    4096 x 4096 matvec, the decode layer with fp32 activations and in Q4_0 (under `.int(8)` both as recipe computes it, over
    the Q8_0 re-encode, and as the direct dot over the stored nibbles), `down` and the LM head under recipe's `.int(8)`,
    and the batched tensor-core product at 16 / 64 / 512 tokens with fp32 and int8 activations."""
    out = {}
    gen = torch.Generator(device=device)
    gen.manual_seed(5)
    stream = torch.cuda.current_stream()
    peak, _ = measured_peak_gbs()

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

    def matvec_line(t, rows, cols, mode, copies, label, weights=None):
        ws = weights or quantised(t, rows, cols, copies)
        x = torch.randn(cols, generator=gen, device=device)
        y = torch.empty(rows, device=device)
        ctx.reserve(rows, cols, 1)
        us = graph_time(lambda i: ctx.matvec(ws[i % len(ws)], x, y, act_mode=mode, step=32), 8 * len(ws))
        nbytes = algo_bytes(ws[0].type, rows, cols)
        out[label] = {"us": us, "GBps": nbytes / us / 1e3, "frac_of_hbm_measured": nbytes / us / 1e3 / peak, "algorithmic_bytes": nbytes}
        return ws

    # cfg 1: Q8_0 4096 x 4096, eight copies in rotation (143 MB: larger than L2)
    for w in matvec_line(Q8_0, 4096, 4096, rq.ACT_INT8, 8, "q8_0_4096x4096_int8_batch1"):
        w.free()
    # fp32 activations (the `.fp` handling, and every expert bank's)
    for w in matvec_line(Q4_K, 14336, 4096, rq.ACT_FLOAT, 4, "q4k_14336x4096_float_batch1"):
        w.free()
    for w in matvec_line(Q6_K, 4096, 14336, rq.ACT_FLOAT, 4, "q6k_4096x14336_float_batch1"):
        w.free()
    # the Q4_0 layer's widest projection, and `down`: `.int(8)` as recipe computes it (the Q8_0 re-encode made at load) and
    # the direct dot over the stored blocks
    for t, rows, cols, name in ((Q4_0, 14336, 4096, "q4_0_14336x4096"), (Q6_K, 4096, 14336, "q6k_4096x14336")):
        stored = matvec_line(t, rows, cols, rq.ACT_INT8, 4, f"{name}_int8_direct_batch1")
        reenc = [ctx.int8_weight(w) for w in stored]
        for w in stored:
            w.free()
        matvec_line(Q8_0, rows, cols, rq.ACT_INT8, 4, f"{name}_int8_recipe_q8_0_reencode_batch1", weights=reenc)
        for w in reenc:
            w.free()
    # `.int(4)`: storage Q4_1 made at load from the Q4_K tensor, int8 records against its four-bit codes (a plain warp-per-row kernel)
    stored = quantised(Q4_K, 14336, 4096, 4)
    four = [ctx.int4_weight(w) for w in stored]
    for w in stored:
        w.free()
    matvec_line(rq.Q4_1, 14336, 4096, rq.ACT_INT8, 4, "q4k_14336x4096_int4_recipe_q4_1_reencode_batch1", weights=four)
    for w in four:
        w.free()
    # cfg 5: the batched product on the tensor cores, fp32 and int8 activations, each call's launches captured in a graph
    for name, t, rows, cols in (("q4k_14336x4096", Q4_K, 14336, 4096), ("q6k_4096x14336", Q6_K, 4096, 14336)):
        ws = quantised(t, rows, cols, 4)
        ctx.reserve(rows, cols, 512)
        for tokens in (16, 64, 512):
            xb = torch.randn(tokens, cols, generator=gen, device=device)
            yb = torch.empty(tokens, rows, device=device)
            for mode, tag in ((rq.ACT_FLOAT, ""), (rq.ACT_INT8, "_int8")):
                us = graph_time(lambda i: ctx.matmul(ws[i % 4], xb, yb, act_mode=mode, step=32), 8)
                flops = 2.0 * rows * cols * tokens
                hbm_us = algo_bytes(t, rows, cols, tokens) / peak / 1e3
                out[f"matmul_{name}_tokens{tokens}{tag}"] = {"us": us, "TFLOPs_useful": flops / us / 1e6, "hbm_time_us": hbm_us}
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
