#!/usr/bin/env python
"""Benchmark of the W4A16 quantized-linear engine.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Prints ONE JSON line.  A "step" is one pass of the hot path over one batch of synthetic
input: every projection of the workload at every batch size M, over enough distinct
layers that the weights of a step (>= 250 MB) cannot stay in the 126 MB L2.

  metric  weight-HBM GB/s = algorithmic weight bytes (N*K/2 + N*ceil(K/64)*4.5 per layer)
          streamed per second, whole job (all ranks)
  value   device-resident inputs, the step replayed as one CUDA graph, CUDA events
  e2e     the same step through the public operator (QuantizedLinear.forward; captured into a CUDA
          graph as a serving loop does, the eager figure beside it) with
          x copied from pinned host memory and y copied back for every call (copies on side
          streams, pipelined against the launches in --e2e-groups groups)
  roofline, cpu_baseline, clocks, gpu_launches: see the keys' comments below

Workloads (shapes are N x K of synthetic projections, weights ~ N(0, sigma^2) quantized
by QuantizedLinear.from_float(group_size=64), x ~ N(0,1) FP16):
  qwen3-0.6b-decode  28 layers x {4096x1024, 1024x2048, 6144x1024, 1024x3072}, M in 1,2,4,8
  qwen3-8b-layer      3 layers x {6144x4096, 4096x4096, 24576x4096, 4096x12288}, M in 1,16
  llama3-70b-mlp      1 layer  x {57344x8192, 8192x28672}, M in 1,8, rows sharded over ranks

With N > 1 (launched under torchrun, one rank per GPU) the first two workloads run one
replica of the projection set per rank (weak scaling: rank r owns rows [r*N,(r+1)*N) of a
P-times wider layer, no exchange); llama3-70b-mlp splits each layer's rows over the ranks
(strong scaling) and `--gather` adds the NCCL all-gather of the output slices.

`--impl reference` times the CPU restatement of the reference's own CPU route (the oracle,
torch FP32 matmul on all host threads) on a bounded sample of the same workload.
"""
import argparse
import copy
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch

WORKLOADS = {
    "qwen3-0.6b-decode": {"shapes": [("qkv", 4096, 1024), ("o", 1024, 2048), ("gate_up", 6144, 1024),
                                     ("down", 1024, 3072)],
                          "layers": 28, "ms": [1, 2, 4, 8], "detail_ms": [16, 512], "sigma": 0.02, "seed": 1000,
                          "shard": False},
    "qwen3-8b-layer": {"shapes": [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 24576, 4096),
                                  ("down", 4096, 12288)],
                       "layers": 3, "ms": [1, 16], "detail_ms": [8, 512, 2048], "sigma": 0.02, "seed": 2000,
                       "shard": False},
    "llama3-70b-mlp": {"shapes": [("gate_up", 57344, 8192), ("down", 8192, 28672)],
                       "layers": 1, "ms": [1, 8], "detail_ms": [16, 256, 4096], "sigma": 0.015, "seed": 3000,
                       "shard": True},
}
FALLBACK_HBM_GBS = 6650.0


def weight_bytes(n, k):
    """Algorithmic weight bytes of one layer: 4-bit codes + FP32 step + 4-bit zero point per group."""
    return n * k / 2 + n * ((k + 63) // 64) * 4.5


def io_bytes(m, n, k):
    return 2 * m * k + 2 * m * n


def measured_hbm_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (KeyError, ValueError):
            pass
    return FALLBACK_HBM_GBS, "fallback"


def measured_tensor_peak():
    """Dense tensor roofline for the prefill rows: the measured cuBLAS bf16 burst (a kernel timed
    alone), else the profiling recipe's fallback."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            return float(json.loads(path.read_text())["bf16_tflops"]), "measured"
        except (KeyError, ValueError):
            pass
    return 1590.0, "fallback"


def prefill_roofline(detail):
    """Tensor-bound roofline of the GEMM kernel from the per-shape table: the largest prefill
    problem measured (flops = 2*M*N*K per launch / CUDA-event time of the launch)."""
    rows = [r for rows in (detail or {}).values() for r in rows if r["M"] >= 512 and r["kernel"] == "b200_tcgen05"]
    if not rows:
        return None
    top = max(rows, key=lambda r: r["M"] * r["N"] * r["K"])
    peak, kind = measured_tensor_peak()
    return {"bound": "tensor", "achieved": top["TFLOPS"], "peak": peak, "unit": "TFLOP/s",
            "frac": round(top["TFLOPS"] / peak, 4), "traffic": None, "peak_kind": kind,
            "kernel": "w4a16_gemm_pair_kernel", "problem": f"{top['N']}x{top['K']}, M={top['M']}",
            "all_prefill_rows_frac": {f"{r['proj']} {r['N']}x{r['K']} M={r['M']}": round(r["TFLOPS"] / peak, 3) for r in rows}}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            self.thread.join(timeout=2)

    def hold_load(self, run, sync, min_samples, limit_s):
        """Keep the GPU under the benchmark's own load (`run` = one step, `sync` = wait for it) until
        `min_samples` samples have arrived or `limit_s` seconds have passed: nvidia-smi needs longer to
        start than a short timed region lasts, so the region is embedded in a longer stretch of the
        same back-to-back replays and every sample is taken under that load."""
        if self.proc is None:
            return
        t_end = time.monotonic() + limit_s
        while len(self.lines) < min_samples and time.monotonic() < t_end:
            for _ in range(8):
                run()
            sync()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            reasons.update(n for n, v in zip(names, parts[2:]) if v == "Active")
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm),
                "window": "back-to-back replays of the step from before the first sample until after the last; "
                          "the timed region lies inside"}


# ----------------------------------------------------------------------------------------------
# workload construction
# ----------------------------------------------------------------------------------------------
def build_layers(spec, rank, world, device):
    """[(name, n_local, k, layer)] per layer index; weights are seeded per (layer, shape, rank)."""
    import dandan_ops_b200 as ops
    from dandan_ops_b200.sharded import shard_rows

    out = []
    for li in range(spec["layers"]):
        row = []
        for si, (name, n, k) in enumerate(spec["shapes"]):
            gen = torch.Generator(device=device)
            gen.manual_seed(spec["seed"] + 100 * li + si + 7919 * rank)   # a stream per (layer, shape, rank)
            rows = n
            if spec["shard"]:
                start, stop = shard_rows(n, world, rank)
                rows = stop - start
            if rows == 0:
                row.append((name, 0, k, None))
                continue
            w = (torch.randn(rows, k, generator=gen, device=device) * spec["sigma"]).half()
            row.append((name, rows, k, ops.QuantizedLinear.from_float(w, group_size=64)))
            del w
        out.append(row)
    return out


def make_inputs(spec, device, pinned=False):
    xs = {}
    gen = torch.Generator().manual_seed(spec["seed"] + 5)
    for m in spec["ms"]:
        for k in sorted({k for _, _, k in spec["shapes"]}):
            x = torch.randn(m, k, generator=gen).half()
            xs[(m, k)] = x.pin_memory() if pinned else x.to(device)
    return xs


def run_gpu(args, rank, world, local_rank):
    import torch.distributed as dist
    from dandan_ops_b200 import _native

    spec = WORKLOADS[args.workload]
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    _native.load()

    layers = build_layers(spec, rank, world, device)
    x_dev = make_inputs(spec, device)
    x_host = make_inputs(spec, device, pinned=True)
    calls = [(m, name, n, k, layer) for m in spec["ms"] for row in layers for (name, n, k, layer) in row
             if layer is not None]
    step_weight_bytes = sum(weight_bytes(n, k) for _, _, n, k, _ in calls)
    step_alg_bytes = step_weight_bytes + sum(io_bytes(m, n, k) for m, _, n, k, _ in calls)
    native_resident = sum(layer.native_bytes for row in layers for (_, _, _, layer) in row if layer is not None)

    gather_layers = None
    if args.gather and spec["shard"] and world > 1:
        from dandan_ops_b200.sharded import ColumnShardedLinear
        gather_layers = {id(layer): ColumnShardedLinear(layer, out_features=n_full, rank=rank, world_size=world)
                         for row in layers for ((name, n, k, layer), (_, n_full, _)) in zip(row, spec["shapes"])
                         if layer is not None}

    def one_step():
        outs = None
        for m, _, n, k, layer in calls:
            y = layer(x_dev[(m, k)])
            if gather_layers is not None:
                y = gather_layers[id(layer)].gather(y)
            outs = y
        return outs

    stream = torch.cuda.Stream(device)
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        before = _native.launch_count()
        one_step()
        launches_per_step = _native.launch_count() - before
        for _ in range(2):
            one_step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        use_graph = gather_layers is None       # the NCCL gather is launched eagerly, not captured
        if use_graph:
            with torch.cuda.graph(graph, stream=stream):
                one_step()
            replay = graph.replay
        else:
            replay = one_step

        def sync_all():
            stream.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        for _ in range(max(args.warmup, 3)):
            replay()
        sync_all()
        with ClockSampler(local_rank) as clocks:
            # graph replays only: a rank-dependent number of eager NCCL gathers would desynchronize the ranks
            if use_graph:
                clocks.hold_load(replay, stream.synchronize, 1, 8.0)
                first = len(clocks.lines)
            sync_all()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(args.steps):
                replay()
            e1.record(stream)
            sync_all()
            if use_graph:
                clocks.hold_load(replay, stream.synchronize, first + 3, 2.0)
            else:
                time.sleep(0.15)
        gpu_ms = e0.elapsed_time(e1)

        # end to end: every call's x starts in pinned host memory and every call's y ends there.  The
        # copies are batched: one H2D of all inputs of the step, the public API call per linear on
        # views of that buffer, one gather + one D2H of all outputs.
        in_sizes = [m * k for m, _, _, k, _ in calls]
        out_sizes = [m * n for m, _, n, _, _ in calls]
        x_all_host = torch.empty(sum(in_sizes), dtype=torch.float16).pin_memory()
        offset = 0
        for (m, _, _, k, _), size in zip(calls, in_sizes):
            x_all_host[offset:offset + size].copy_(x_host[(m, k)].reshape(-1))
            offset += size
        x_all_dev = torch.empty_like(x_all_host, device=device)
        x_views, offset = [], 0
        for (m, _, _, k, _), size in zip(calls, in_sizes):
            x_views.append(x_all_dev[offset:offset + size].view(m, k))
            offset += size
        y_all_dev = torch.empty(sum(out_sizes), dtype=torch.float16, device=device)
        y_all_host = torch.empty(sum(out_sizes), dtype=torch.float16).pin_memory()

        # The step is cut into groups of calls: the inputs of every group are copied on one side stream,
        # the outputs on another, so that a group's copies overlap the launches of its neighbours
        # (PCIe is full duplex).  Every byte still crosses in every step, inside the timed region.
        n_groups = max(1, min(args.e2e_groups, len(calls)))
        bounds = [len(calls) * g // n_groups for g in range(n_groups + 1)]
        in_off = [sum(in_sizes[:i]) for i in range(len(calls) + 1)]
        out_off = [sum(out_sizes[:i]) for i in range(len(calls) + 1)]
        copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)

        def e2e_step():
            main = torch.cuda.current_stream()
            copy_in.wait_stream(main)
            arrived = []
            with torch.cuda.stream(copy_in):
                for g in range(n_groups):
                    lo, hi = in_off[bounds[g]], in_off[bounds[g + 1]]
                    x_all_dev[lo:hi].copy_(x_all_host[lo:hi], non_blocking=True)
                    arrived.append(torch.cuda.Event())
                    arrived[-1].record(copy_in)
            for g in range(n_groups):
                main.wait_event(arrived[g])
                outs = [calls[i][4](x_views[i]).reshape(-1) for i in range(bounds[g], bounds[g + 1])]
                lo, hi = out_off[bounds[g]], out_off[bounds[g + 1]]
                torch.cat(outs, out=y_all_dev[lo:hi])
                done = torch.cuda.Event()
                done.record(main)
                copy_out.wait_event(done)
                with torch.cuda.stream(copy_out):
                    y_all_host[lo:hi].copy_(y_all_dev[lo:hi], non_blocking=True)
            main.wait_stream(copy_out)

        def timed(fn, steps):
            fn()
            sync_all()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(stream)
            for _ in range(steps):
                fn()
            t1.record(stream)
            sync_all()
            return t0.elapsed_time(t1) / steps

        e2e_steps = max(1, min(args.steps, 5))
        e2e_eager_ms = timed(e2e_step, e2e_steps)            # one eager Python call per linear
        # The way a serving loop runs a decode step: the same calls and the same copies captured
        # once through the public API into a CUDA graph (the copies become memcpy nodes on the
        # pinned buffers) and replayed; the host refreshes x_host in place between replays.
        e2e_ms = e2e_eager_ms * e2e_steps
        e2e_mode = "eager"
        if use_graph:
            e2e_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(e2e_graph, stream=stream):
                e2e_step()
            e2e_ms = timed(e2e_graph.replay, e2e_steps) * e2e_steps
            e2e_mode = "cuda_graph"

    times = torch.tensor([gpu_ms / args.steps, e2e_ms / e2e_steps, e2e_eager_ms], dtype=torch.float64, device=device)
    bytes_all = torch.tensor([step_weight_bytes, step_alg_bytes], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(bytes_all, op=dist.ReduceOp.SUM)
    ms_per_step, e2e_ms_per_step, e2e_eager_ms_per_step = (float(v) for v in times.cpu())
    weight_total, alg_total = (float(v) for v in bytes_all.cpu())

    detail = None
    if rank == 0 and not args.no_detail:
        detail = {args.workload: per_shape_detail(spec, layers, x_dev, stream, device)}
        if world == 1 and not args.workload_only:
            # the other benchmark configurations, one table each (decode GB/s and prefill TFLOP/s)
            for other in sorted(WORKLOADS):
                if other == args.workload:
                    continue
                ospec = dict(WORKLOADS[other])
                ospec["layers"] = min(ospec["layers"], 2)
                olayers = build_layers(ospec, 0, 1, device)
                detail[other] = per_shape_detail(ospec, olayers, make_inputs(ospec, device), stream, device)
                del olayers
                torch.cuda.empty_cache()
    cpu = cpu_baseline(spec, sample_seconds=args.cpu_seconds) if (rank == 0 and world == 1 and not args.no_cpu) else None

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        # per launch: one rank's algorithmic bytes of a step / its launches, over the average launch time
        launches = launches_per_step
        achieved = (step_alg_bytes / launches) / (ms_per_step * 1e-3 / launches) / 1e9
        result = {
            "metric": "w4a16_decode_weight_hbm_GBps", "value": round(weight_total / (ms_per_step * 1e-3) / 1e9, 2),
            "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "strong" if spec["shard"] else "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": args.workload, "layers": spec["layers"], "batch_sizes": spec["ms"],
                       "arithmetic": "u4 codes, exact f16 weights, f16 activations, f32 accumulate, f16 output",
                       "shapes_NxK": [f"{n}x{k}" for _, n, k in spec["shapes"]],
                       "linears_per_step": len(calls), "weight_bytes_per_step_per_gpu": int(step_weight_bytes),
                       "native_image_bytes_resident_per_gpu": int(native_resident),
                       "cache": "weights of a step exceed L2 (inputs larger than L2, no flush)",
                       "timing": "step replayed as one CUDA graph" if use_graph else "eager launches",
                       "gather": bool(gather_layers)},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4),
                         # ncu (profiles/): DRAM bytes read+written = 1.015 x (tile kernel) / 1.005 x (streaming
                         # kernel) the algorithmic weight bytes of a launch; scaled here to the average launch
                         "traffic": round((step_weight_bytes / launches) * (1.015 if args.workload == "qwen3-0.6b-decode" else 1.005)),
                         "traffic_unit": "bytes per launch", "peak_kind": peak_kind,
                         "kernel": "w4a16_tile_kernel" if args.workload == "qwen3-0.6b-decode" else "w4a16_stream_kernel",
                         "note": "achieved = algorithmic bytes per launch / average launch time over the graph"},
            "cpu_baseline": cpu,
            "e2e": {"value": round(weight_total / (e2e_ms_per_step * 1e-3) / 1e9, 2), "unit": "GB/s",
                    "h2d_bytes_per_step": int(sum(2 * m * k for m, _, _, k, _ in calls)),
                    "d2h_bytes_per_step": int(sum(2 * m * n for m, _, n, _, _ in calls)),
                    "ms_per_step": round(e2e_ms_per_step, 4),
                    "copy_groups": n_groups,
                    "how": (f"the step's calls in {n_groups} groups: each group's inputs pinned host -> device in one copy on a "
                            "side stream, QuantizedLinear.forward per linear, the group's outputs gathered and copied "
                            "device -> pinned host in one copy on a second side stream, so copies overlap the "
                            "neighbouring groups' launches; "
                            + ("captured once through the public API into a CUDA graph and replayed" if e2e_mode == "cuda_graph"
                               else "one eager Python call per linear")),
                    "eager": {"value": round(weight_total / (e2e_eager_ms_per_step * 1e-3) / 1e9, 2),
                              "ms_per_step": round(e2e_eager_ms_per_step, 4),
                              "how": "the same step with one eager Python call per linear"}},
            "gpu_launches": int(launches_per_step * args.steps),
            "clocks": clocks.summary(),
            "roofline_prefill": prefill_roofline(detail),
            "detail": detail,
        }
        print(json.dumps(result))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def per_shape_detail(spec, layers, x_dev, stream, device):
    """Median CUDA-graph replay time of every (projection, M): microseconds, weight GB/s, TFLOPS.
    Decode sizes: each graph walks >= 256 MB of distinct layers once, so every launch streams its
    weights from HBM in every replay.  Prefill sizes: one pass over the column, L2 flushed (a 256 MB
    memset, untimed) before every replay.  `detail_ms` adds batch sizes that are not
    part of the timed step, among them the prefill sizes that run on the tcgen05 GEMM."""
    out = []
    gen = torch.Generator().manual_seed(spec["seed"] + 6)
    all_ms = sorted(set(spec["ms"]) | set(spec.get("detail_ms", [])))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)      # larger than L2
    with torch.cuda.stream(stream):
        # Decode sizes of every projection first, the prefill sizes last: seconds of GEMM at the
        # power cap lower the SM clock for a while, which would tax whatever is timed right after.
        for prefill in (False, True):
            for si, (name, n_full, k) in enumerate(spec["shapes"]):
                column = [row[si] for row in layers if row[si][3] is not None]
                if not column:
                    continue
                n = column[0][1]
                if not prefill:
                    # Decode sizes are timed over >= 256 MB of distinct weights (copies of the column's layers),
                    # so that a replay streams every layer from HBM, as the step does, instead of finding a
                    # small column (28 x 2.4 MB) still in L2 from the previous replay.
                    need = int(256e6 // max(1.0, weight_bytes(n, k))) + 1
                    base = list(column)
                    while len(column) < min(need, 160):
                        name_, n_, k_, layer_ = base[len(column) % len(base)]
                        column.append((name_, n_, k_, copy.deepcopy(layer_)))
                for m in all_ms:
                    if (m > 64) != prefill:
                        continue
                    reps = 1
                    x = x_dev.get((m, k))
                    if x is None:
                        x = torch.randn(m, k, generator=gen).half().to(device)
                    for _, _, _, layer in column:
                        layer(x)
                    stream.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=stream):
                        for _ in range(reps):
                            for _, _, _, layer in column:
                                layer(x)
                    samples = []
                    for _ in range(7):
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        if prefill:
                            flush.zero_()
                        e0.record(stream)
                        graph.replay()
                        e1.record(stream)
                        stream.synchronize()
                        samples.append(e0.elapsed_time(e1) * 1e3 / (reps * len(column)))
                    us = statistics.median(samples)
                    out.append({"proj": name, "N": n, "K": k, "M": m, "us": round(us, 2),
                                "kernel": layer.execution_info(x)["implementation"],
                                "weight_GBps": round(weight_bytes(n, k) / us / 1e3, 1),
                                "TFLOPS": round(2.0 * m * n * k / us / 1e6, 2)})
    out.sort(key=lambda r: ([s[0] for s in spec["shapes"]].index(r["proj"]), r["M"]))
    return out


# ----------------------------------------------------------------------------------------------
# CPU baseline / reference arm: the oracle's restatement of the reference's CPU route
# ----------------------------------------------------------------------------------------------
def cpu_state(n, k, sigma, seed):
    from oracle import w4a16_oracle as oracle

    gen = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, k, generator=gen) * sigma).half()
    codes, step, zero = oracle.quantize(w.numpy())
    return torch.from_numpy(oracle.pack(codes)), torch.from_numpy(step), torch.from_numpy(zero)


def cpu_pass(spec, states, xs):
    """One pass over one layer's projections at every M on the host.  Returns weight bytes covered."""
    from oracle import w4a16_oracle as oracle

    covered = 0.0
    for (name, n, k), (words, step, zero) in zip(spec["shapes"], states):
        for m in spec["ms"]:
            oracle.torch_forward(xs[(m, k)], words, step, zero, k)
            covered += weight_bytes(n, k)
    return covered


def cpu_baseline(spec, sample_seconds=15.0):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    shapes = spec["shapes"]
    if max(n * k for _, n, k in shapes) > 200e6:      # bound the sample: quarter-height slices of huge layers
        shapes = [(name, n // 8, k) for name, n, k in shapes]
    small = dict(spec, shapes=shapes)
    states = [cpu_state(n, k, spec["sigma"], spec["seed"] + i) for i, (_, n, k) in enumerate(shapes)]
    gen = torch.Generator().manual_seed(spec["seed"] + 5)
    xs = {(m, k): torch.randn(m, k, generator=gen).half() for m in spec["ms"] for k in {k for _, _, k in shapes}}
    cpu_pass(small, states, xs)                        # warm-up
    covered, t0, passes = 0.0, time.perf_counter(), 0
    while passes < 1 or (time.perf_counter() - t0 < sample_seconds and passes < 50):
        covered += cpu_pass(small, states, xs)
        passes += 1
    elapsed = time.perf_counter() - t0
    return {"value": round(covered / elapsed / 1e9, 4), "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"{passes} passes over one layer's projections {[f'{n}x{k}' for _, n, k in shapes]} "
                      f"at M={spec['ms']} ({elapsed:.1f} s, torch FP32 matmul restatement of the reference CPU route)"}


def run_reference(args, rank, world):
    if rank != 0:
        return
    spec = WORKLOADS[args.workload]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    shapes = spec["shapes"]
    if max(n * k for _, n, k in shapes) > 200e6:
        shapes = [(name, n // 8, k) for name, n, k in shapes]
    small = dict(spec, shapes=shapes)
    states = [cpu_state(n, k, spec["sigma"], spec["seed"] + i) for i, (_, n, k) in enumerate(shapes)]
    gen = torch.Generator().manual_seed(spec["seed"] + 5)
    xs = {(m, k): torch.randn(m, k, generator=gen).half() for m in spec["ms"] for k in {k for _, _, k in shapes}}
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_pass(small, states, xs)
    t0 = time.perf_counter()
    covered = 0.0
    for _ in range(args.steps):
        covered += cpu_pass(small, states, xs)
    elapsed = time.perf_counter() - t0
    value = round(covered / elapsed / 1e9, 4)
    sample = (f"each step = one layer's projections {[f'{n}x{k}' for _, n, k in shapes]} at M={spec['ms']} "
              f"on {cores} host threads")
    print(json.dumps({
        "impl": "reference", "metric": "w4a16_decode_weight_hbm_GBps", "value": value, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(elapsed / args.steps * 1e3, 3), "higher_is_better": True,
        "scaling": "strong" if spec["shard"] else "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": args.workload, "batch_sizes": spec["ms"],
                   "shapes_NxK": [f"{n}x{k}" for _, n, k in shapes]},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="qwen3-0.6b-decode")
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--gather", action="store_true", help="all-gather output slices (sharded workload, N>1)")
    ap.add_argument("--no-detail", action="store_true", help="skip the per-shape table")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--workload-only", action="store_true", help="per-shape table for the chosen workload only")
    ap.add_argument("--e2e-groups", type=int, default=32, help="copy/launch groups of the end-to-end step (1 = one copy each way)")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world != args.gpus and args.gpus > 1:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the package has no CPU compute path")
    run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
