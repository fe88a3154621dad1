#!/usr/bin/env python
"""Benchmark of the W4A16 quantized-linear engine.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Prints ONE JSON line.  A "step" is one pass of the hot path over one batch of synthetic input:
every projection of the workload at every decode batch size M, over enough distinct layers that
the weights a rank streams per step (>= 300 MB) cannot stay in the 126 MB L2.

  metric  weight-HBM GB/s = algorithmic weight bytes (N*K/2 + N*ceil(K/64)*4.5 per layer) streamed per
          second, whole job (all ranks)
  value   device-resident inputs, the step replayed as one CUDA graph, CUDA events, max over ranks
  e2e     the same step through the public operator (QuantizedLinear.forward, or the column-sharded
          layer's forward(gather=True) at N > 1) with x copied from pinned host memory and y copied
          back inside the timed region
  roofline, roofline_prefill, floor_us, warm, parity, cpu_baseline, clocks, gpu_launches: see below

Workloads (N x K of synthetic projections, weights ~ N(0, sigma^2) quantized by
QuantizedLinear.from_float(group_size=64), x ~ N(0,1) FP16):
  llama3-70b-mlp (default)  6 layers x {57344x8192, 8192x28672}, M in 1,8.  With N > 1 ranks every
                            layer's rows (output columns) are split over the ranks - strong scaling -
                            and the output slices are gathered over NVLink inside the timed region:
                            projection and gather are ONE launch per linear (the streaming kernel sends
                            every finished tile to the peers' mailboxes and collects theirs;
                            --separate-gather runs the projection and then the gather kernel,
                            --no-gather leaves the slices where they are)
  qwen3-8b-layer            3 layers x {6144x4096, 4096x4096, 24576x4096, 4096x12288}, M in 1,16
  qwen3-0.6b-decode         28 layers x {4096x1024, 1024x2048, 6144x1024, 1024x3072}, M in 1,2,4,8
(the last two run one replica per rank at N > 1: weak scaling, no exchange)

`--impl reference` times the reference's own CPU route on the host cores: the reference package when
it can be imported (a checkout named by the environment variable B2_REFERENCE_ROOT), else the oracle's
restatement of it.
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

import numpy as np
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
                       "layers": 6, "ms": [1, 8], "detail_ms": [16, 256, 4096], "sigma": 0.015, "seed": 3000,
                       "shard": True},
}
FALLBACK_HBM_GBS = 6650.0
NOMINAL_HBM_GBS, NOMINAL_FP16_TFLOPS = 8000.0, 2250.0


def weight_bytes(n, k):
    """Algorithmic weight bytes of one layer: 4-bit codes + FP32 step + 4-bit zero point per group."""
    return n * k / 2 + n * ((k + 63) // 64) * 4.5


def io_bytes(m, n, k):
    return 2 * m * k + 2 * m * n


def measured_peak(key, fallback):
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            return float(json.loads(path.read_text())[key]), "measured"
        except (KeyError, ValueError):
            pass
    return fallback, "fallback"


def dram_traffic_factor(kernel):
    """DRAM bytes (read + written) per algorithmic weight byte of a launch, as ncu measured it for
    `kernel`: the table lives in profiles/dram_traffic_per_kernel.md (| kernel | factor | capture |)."""
    path = ROOT / "profiles" / "dram_traffic_per_kernel.md"
    if not path.is_file():
        return None
    for line in path.read_text().splitlines():
        cells = [c.strip() for c in line.strip().strip("|").split("|")]
        if len(cells) >= 2 and cells[0].strip("`") == kernel:
            try:
                return float(cells[1])
            except ValueError:
                return None
    return None


def prefill_roofline(detail):
    """Tensor-bound roofline of the GEMM kernel from the per-shape table: the largest prefill
    problem measured (flops = 2*M*N*K per launch / CUDA-event time of the launch)."""
    rows = [r for rows in (detail or {}).values() for r in rows if r["M"] >= 512 and r["kernel"] == "b200_tcgen05"]
    if not rows:
        return None
    top = max(rows, key=lambda r: r["M"] * r["N"] * r["K"])
    peak, kind = measured_peak("bf16_tflops", 1590.0)
    return {"bound": "tensor", "achieved": top["TFLOPS"], "peak": peak, "unit": "TFLOP/s",
            "frac": round(top["TFLOPS"] / peak, 4), "frac_of_nominal_2250": round(top["TFLOPS"] / NOMINAL_FP16_TFLOPS, 4),
            "traffic": None, "peak_kind": kind,
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
    """[(name, n_local, k, layer, n_full)] per layer index; weights are seeded per (layer, shape, rank)."""
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
                row.append((name, 0, k, None, n))
                continue
            w = (torch.randn(rows, k, generator=gen, device=device) * spec["sigma"]).half()
            row.append((name, rows, k, ops.QuantizedLinear.from_float(w, group_size=64), n))
            del w
        out.append(row)
    return out


def build_fp16_step_layers(spec, device, layers=2):
    """The same shapes with a state built directly, as the stress configuration builds it: uniform codes and
    zero points, log-normal steps rounded to FP16 (what checkpoints with FP16 scales hold).  The module then
    sets B2_FLAG_FP16_STEPS and the kernels run the FP16-only dequantization."""
    import dandan_ops_b200 as ops

    out = []
    for li in range(layers):
        row = []
        for si, (name, n, k) in enumerate(spec["shapes"]):
            gen = torch.Generator(device=device)
            gen.manual_seed(spec["seed"] + 9000 + 100 * li + si)
            groups = (k + 63) // 64
            codes = torch.randint(0, 16, (n, k), generator=gen, dtype=torch.uint8, device=device)
            zero = torch.randint(0, 16, (n, groups), generator=gen, dtype=torch.int32, device=device)
            step = torch.exp(torch.randn(n, groups, generator=gen, device=device) * 0.5 - 5.0).half().float()
            layer = ops.QuantizedLinear(ops.pack_int4(codes), step, zero, in_features=k)
            assert layer._image_flags & 1
            row.append((name, n, k, layer, n))
            del codes
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


def time_graph(graph, stream, sync_all, steps):
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        graph.replay()
    e1.record(stream)
    sync_all()
    return e0.elapsed_time(e1) / steps


def capture(fn, stream):
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        fn()
    return graph


def parity_check(calls, x_dev, run_call, rank, world, gathered):
    """Outside the timed region: every timed linear on sampled output columns against the CPU oracle
    (reference acceptance rule |y - y_ref| <= 2e-3 + 2e-3|y_ref|).  At N > 1 with the gather on, rank 0
    checks the GATHERED [M, N] it holds against the oracle on columns sampled from every rank's rows."""
    import torch.distributed as dist

    import cases
    from oracle import w4a16_oracle as oracle

    worst = {"max_abs": 0.0, "relative_l2": 0.0, "mismatch_fraction": 0.0, "bound_ratio": 0.0}
    checked = 0
    for call in calls:
        m, name, n_local, k, layer, n_full, start = call["m"], call["name"], call["n"], call["k"], call["layer"], call["n_full"], call["start"]
        pick = torch.linspace(0, max(n_local - 1, 0), steps=min(48, n_local)).long().unique()
        if layer is None:                               # a rank without rows of this layer
            state = [np.zeros((0, (k + 7) // 8), np.int32), np.zeros((0, (k + 63) // 64), np.float32), np.zeros((0, (k + 63) // 64), np.int32)]
        else:
            state = [t[pick.to(t.device)].cpu().numpy() for t in (layer.packed_weight, layer.scales, layer.zeros)]
        cols = (pick + start).numpy()
        y = run_call(call)
        torch.cuda.synchronize()
        if gathered:
            parts = [None] * world if rank == 0 else None
            dist.gather_object((cols, state), parts, dst=0)
            if rank != 0:
                continue
            cols = np.concatenate([p[0] for p in parts])
            state = [np.concatenate([p[1][i] for p in parts]) for i in range(3)]
            got = y[:, torch.from_numpy(cols).to(y.device)].cpu().numpy()
        else:
            got = y[:, pick.to(y.device)].cpu().numpy()
        ref = oracle.linear(x_dev[(m, k)].cpu().numpy(), state[0], state[1], state[2], k)
        metrics = cases.error_metrics(got, ref)
        for key in worst:
            worst[key] = max(worst[key], metrics[key])
        checked += 1
    if rank != 0 and gathered:
        return None
    return {"ok": worst["bound_ratio"] <= 1.0, "linears_checked": checked, "columns_per_linear": "48 per rank, evenly spaced",
            "rule": "|y - y_ref| <= 2e-3 + 2e-3*|y_ref| against the CPU oracle of the reference's CPU route",
            "checked_tensor": "gathered [M, N] on rank 0" if gathered else "this rank's output",
            **{k: float(f"{v:.4g}") for k, v in worst.items()}}


def run_gpu(args, rank, world, local_rank):
    import torch.distributed as dist
    from dandan_ops_b200 import _native
    from dandan_ops_b200.sharded import shard_rows

    spec = WORKLOADS[args.workload]
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    _native.load()

    layers = build_layers(spec, rank, world, device)
    x_dev = make_inputs(spec, device)
    x_host = make_inputs(spec, device, pinned=True)
    gather_on = bool(spec["shard"] and world > 1 and not args.no_gather)
    arena = None
    if gather_on:
        from dandan_ops_b200.sharded import ColumnShardedLinear, PeerArena
        need = sum(2 * (-(-(m * n_full * 2) // 256) * 256) for m in spec["ms"] for row in layers for (_, _, _, _, n_full) in row)
        arena = PeerArena(need + (1 << 20))      # slices up to 1 MB travel as polled packets (the decode sizes)
    calls = []
    for li, row in enumerate(layers):
        for (name, n, k, layer, n_full) in row:
            if layer is None and not gather_on:
                continue
            start = shard_rows(n_full, world, rank)[0] if spec["shard"] else 0
            sharded = (ColumnShardedLinear(layer, out_features=n_full, rank=rank, world_size=world).attach_arena(arena)
                       if gather_on else None)
            if sharded is not None:
                sharded.fuse_gather = not args.separate_gather
            for m in spec["ms"]:
                calls.append({"m": m, "name": name, "n": n, "k": k, "layer": layer, "n_full": n_full, "start": start,
                              "li": li, "sharded": sharded})
    calls.sort(key=lambda c: c["m"])                  # all layers at M = 1, then at the next batch size, ...
    step_weight_bytes = sum(weight_bytes(c["n"], c["k"]) for c in calls)
    step_alg_bytes = step_weight_bytes + sum(io_bytes(c["m"], c["n"], c["k"]) for c in calls)
    native_resident = sum(layer.native_bytes for row in layers for (_, _, _, layer, _) in row if layer is not None)

    def run_call(c, x=None):
        x = x_dev[(c["m"], c["k"])] if x is None else x
        if gather_on:
            return c["sharded"](x, gather=True)
        return c["layer"](x)

    def one_step():
        out = None
        for c in calls:
            out = run_call(c)
        return out

    def proj_step():                                   # the projections alone (no exchange)
        for c in calls:
            if c["layer"] is not None:
                c["layer"](x_dev[(c["m"], c["k"])])

    stream = torch.cuda.Stream(device)
    stream.wait_stream(torch.cuda.current_stream())

    def sync_all():
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        before = _native.launch_count()
        one_step()
        launches_per_step = _native.launch_count() - before
        before = _native.launch_count()
        proj_step()
        proj_launches = _native.launch_count() - before
        for _ in range(2):
            one_step()
        sync_all()
        graph = capture(one_step, stream)
        proj_graph = graph if not gather_on else capture(proj_step, stream)

        def gather_step():                             # the exchange alone: every linear's gather launch, no projection
            for c in calls:
                sl = c["sharded"]
                full, ptrs = sl.arena.output((id(sl), 0), c["m"], c["n_full"])
                _native.gather(ptrs, sl.arena.flag_ptrs, sl.arena.mailbox_slice_bytes, rank, c["m"], c["n_full"], c["n_full"],
                               sl.rows_per_rank)
        gather_graph = capture(gather_step, stream) if gather_on else None
        floor_graph = capture(lambda: [_native.noop() for _ in range(launches_per_step)], stream)
        warm = max(args.warmup, 3)
        for _ in range(warm):
            graph.replay()
        sync_all()
        with ClockSampler(local_rank) as clocks:
            clocks.hold_load(proj_graph.replay, stream.synchronize, 1, 8.0)    # no exchange while ranks are out of step
            first = len(clocks.lines)
            gpu_ms = time_graph(graph, stream, sync_all, args.steps)
            clocks.hold_load(proj_graph.replay, stream.synchronize, first + 3, 2.0)
        proj_ms = gpu_ms if not gather_on else time_graph(proj_graph, stream, sync_all, args.steps)
        gather_ms = time_graph(gather_graph, stream, sync_all, args.steps) if gather_on else 0.0
        floor_ms = time_graph(floor_graph, stream, sync_all, max(args.steps, 20))

        # ---- end to end: x starts in pinned host memory, y ends there, every step -----------------
        in_sizes = [c["m"] * c["k"] for c in calls]
        out_sizes = [c["m"] * (c["n_full"] if gather_on else c["n"]) for c in calls]
        x_all_host = torch.empty(sum(in_sizes), dtype=torch.float16).pin_memory()
        offset = 0
        for c, size in zip(calls, in_sizes):
            x_all_host[offset:offset + size].copy_(x_host[(c["m"], c["k"])].reshape(-1))
            offset += size
        x_all_dev = torch.empty_like(x_all_host, device=device)
        x_views, offset = [], 0
        for c, size in zip(calls, in_sizes):
            x_views.append(x_all_dev[offset:offset + size].view(c["m"], c["k"]))
            offset += size
        y_all_dev = torch.empty(sum(out_sizes), dtype=torch.float16, device=device)
        y_all_host = torch.empty(sum(out_sizes), dtype=torch.float16).pin_memory()
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
                outs = [run_call(calls[i], x_views[i]).reshape(-1) for i in range(bounds[g], bounds[g + 1])]
                lo, hi = out_off[bounds[g]], out_off[bounds[g + 1]]
                torch.cat(outs, out=y_all_dev[lo:hi])
                done = torch.cuda.Event()
                done.record(main)
                copy_out.wait_event(done)
                with torch.cuda.stream(copy_out):
                    y_all_host[lo:hi].copy_(y_all_dev[lo:hi], non_blocking=True)
            main.wait_stream(copy_out)

        e2e_steps = max(1, min(args.steps, 5))
        e2e_step()
        if gather_on:
            e2e_step()                                  # both output buffers of every sharded layer exist before capture
        sync_all()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        t1.record(stream)
        sync_all()
        e2e_eager_ms = t0.elapsed_time(t1) / e2e_steps   # one eager Python call per linear
        e2e_graph = capture(e2e_step, stream)
        e2e_graph.replay()
        e2e_ms = time_graph(e2e_graph, stream, sync_all, e2e_steps)

        parity = parity_check([c for c in calls if c["li"] == 0], x_dev, run_call, rank, world, gather_on)

    times = torch.tensor([gpu_ms, e2e_ms, e2e_eager_ms, proj_ms, floor_ms, gather_ms], dtype=torch.float64, device=device)
    bytes_all = torch.tensor([step_weight_bytes, step_alg_bytes], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(bytes_all, op=dist.ReduceOp.SUM)
    ms_per_step, e2e_ms_per_step, e2e_eager_ms_per_step, proj_ms_per_step, floor_ms_per_step, gather_ms_per_step = (
        float(v) for v in times.cpu())
    weight_total, alg_total = (float(v) for v in bytes_all.cpu())
    status = _native.status() | (arena.status() if arena is not None else 0)

    detail, warm_table = None, None
    if rank == 0 and not args.no_detail:
        detail = {args.workload: per_shape_detail(spec, layers, x_dev, stream, device, decode_only=world > 1)}
        if world == 1 and not args.workload_only:
            for other in sorted(WORKLOADS):
                if other == args.workload:
                    continue
                ospec = dict(WORKLOADS[other])
                ospec["layers"] = min(ospec["layers"], 2)
                olayers = build_layers(ospec, 0, 1, device)
                detail[other] = per_shape_detail(ospec, olayers, make_inputs(ospec, device), stream, device)
                del olayers
                torch.cuda.empty_cache()
            warm_table = warm_protocol(stream, device)
            fspec = dict(spec)
            flayers = build_fp16_step_layers(fspec, device)
            detail[args.workload + " with FP16-representable steps (B2_FLAG_FP16_STEPS)"] = per_shape_detail(
                fspec, flayers, make_inputs(fspec, device), stream, device)
            del flayers
            torch.cuda.empty_cache()
    cpu = cpu_baseline(spec, sample_seconds=args.cpu_seconds) if (rank == 0 and world == 1 and not args.no_cpu) else None

    if rank == 0:
        peak, peak_kind = measured_peak("hbm_gbs", FALLBACK_HBM_GBS)
        kernel = "w4a16_tile_kernel" if args.workload == "qwen3-0.6b-decode" else "w4a16_stream_kernel"
        # one rank's projection launches: algorithmic bytes per launch / average launch time (CUDA events over
        # the replayed graph of the projections; at N = 1 that graph is the timed step itself)
        achieved = (step_alg_bytes / proj_launches) / (proj_ms_per_step * 1e-3 / proj_launches) / 1e9
        factor = dram_traffic_factor(kernel)
        result = {
            "metric": "w4a16_decode_weight_hbm_GBps", "value": round(weight_total / (ms_per_step * 1e-3) / 1e9, 2),
            "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "strong" if spec["shard"] else "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": args.workload, "layers": spec["layers"], "batch_sizes": spec["ms"],
                       "arithmetic": "u4 codes, exact f16 weights, f16 activations, f32 accumulate, f16 output",
                       "shapes_NxK": [f"{n}x{k}" for _, n, k in spec["shapes"]],
                       "linears_per_step": len(calls), "weight_bytes_per_step_per_gpu": int(step_weight_bytes),
                       "native_image_bytes_resident_per_gpu": int(native_resident),
                       "cache": "weights a rank streams per step exceed L2 (inputs larger than L2, no flush)",
                       "timing": "step replayed as one CUDA graph, CUDA events on the launching stream, max over ranks",
                       "partition": (f"rows of every layer split over {world} ranks" if spec["shard"] and world > 1 else
                                     "whole layers on every rank"),
                       "gather": (None if not gather_on else
                                  "inside the timed region; projection + gather launches per linear: " +
                                  ", ".join(f"{c['name']} M={c['m']}: {c['sharded'].gather_launches(c['m'])}"
                                            for c in calls if c["li"] == 0) +
                                  " (1 = one kernel streams the weights, sends finished tiles to the peers' mailboxes as "
                                  "{word, epoch} packets and collects theirs; 2 = projection, then the gather kernel)")},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "frac_of_nominal_8000": round(achieved / NOMINAL_HBM_GBS, 4),
                         "traffic": None if factor is None else round(step_weight_bytes / proj_launches * factor),
                         "traffic_unit": "bytes per launch", "traffic_source": "profiles/dram_traffic_per_kernel.md (ncu)",
                         "peak_kind": peak_kind, "kernel": kernel,
                         "us_per_launch": round(proj_ms_per_step * 1e3 / proj_launches, 2),
                         "note": "achieved = algorithmic bytes per projection launch / average launch time (CUDA events over "
                                 "the replayed projections of one rank)"},
            "floor_us": {"per_launch": round(floor_ms_per_step * 1e3 / launches_per_step, 3), "launches": launches_per_step,
                         "how": "an empty kernel per launch of the step, captured and replayed the same way"},
            "parity": parity,
            "status_word": status,
            "cpu_baseline": cpu,
            "e2e": {"value": round(weight_total / (e2e_ms_per_step * 1e-3) / 1e9, 2), "unit": "GB/s",
                    "h2d_bytes_per_step": int(sum(2 * s for s in in_sizes)),
                    "d2h_bytes_per_step": int(sum(2 * s for s in out_sizes)),
                    "ms_per_step": round(e2e_ms_per_step, 4),
                    "copy_groups": n_groups,
                    "how": (f"the step's calls in {n_groups} groups: each group's inputs pinned host -> device in one copy on a "
                            "side stream, the public forward per linear" + (" (sharded forward with gather)" if gather_on else "") +
                            ", the group's outputs copied device -> pinned host in one copy on a second side stream; "
                            "captured once through the public API into a CUDA graph and replayed"),
                    "eager": {"value": round(weight_total / (e2e_eager_ms_per_step * 1e-3) / 1e9, 2),
                              "ms_per_step": round(e2e_eager_ms_per_step, 4),
                              "how": "the same step with one eager Python call per linear"}},
            "gpu_launches": int(launches_per_step * args.steps),
            "clocks": clocks.summary(),
            "roofline_prefill": prefill_roofline({k: v for k, v in (detail or {}).items() if "FP16" not in k}),
            "roofline_prefill_fp16_steps": prefill_roofline({k: v for k, v in (detail or {}).items() if "FP16" in k}),
            "warm": warm_table,
            "detail": detail,
        }
        if gather_on:
            result["projection_only"] = {"ms_per_step": round(proj_ms_per_step, 4),
                                         "value": round(weight_total / (proj_ms_per_step * 1e-3) / 1e9, 2), "unit": "GB/s",
                                         "note": "the same step without the gather launches"}
            result["gather_only"] = {"ms_per_step": round(gather_ms_per_step, 4),
                                     "us_per_gather": round(gather_ms_per_step * 1e3 / len(calls), 2),
                                     "note": "the gather launches of the step alone, ranks in lockstep (no projection between them)"}
        print(json.dumps(result))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def per_shape_detail(spec, layers, x_dev, stream, device, decode_only=False):
    """Median CUDA-graph replay time of every (projection, M): microseconds, weight GB/s, TFLOPS.
    Decode sizes: each graph walks >= 256 MB of distinct layers once, so every launch streams its
    weights from HBM in every replay.  Prefill sizes: one pass over the column, L2 flushed (a 256 MB
    memset, untimed) before every replay.  `detail_ms` adds batch sizes that are not
    part of the timed step, among them the prefill sizes that run on the tcgen05 GEMM."""
    out = []
    gen = torch.Generator().manual_seed(spec["seed"] + 6)
    all_ms = sorted(set(spec["ms"]) | set(spec.get("detail_ms", [])))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)      # larger than L2
    hbm_peak, _ = measured_peak("hbm_gbs", FALLBACK_HBM_GBS)
    with torch.cuda.stream(stream):
        # Decode sizes of every projection first, the prefill sizes last: seconds of GEMM at the
        # power cap lower the SM clock for a while, which would tax whatever is timed right after.
        for prefill in ((False,) if decode_only else (False, True)):
            for si, (name, n_full, k) in enumerate(spec["shapes"]):
                column = [row[si][:4] for row in layers if row[si][3] is not None]
                if not column:
                    continue
                n = column[0][1]
                if not prefill:
                    need = int(256e6 // max(1.0, weight_bytes(n, k))) + 1
                    base = list(column)
                    while len(column) < min(need, 160):
                        name_, n_, k_, layer_ = base[len(column) % len(base)]
                        column.append((name_, n_, k_, copy.deepcopy(layer_)))
                else:
                    column = column[:2]
                for m in all_ms:
                    if (m > 64) != prefill:
                        continue
                    x = x_dev.get((m, k))
                    if x is None:
                        x = torch.randn(m, k, generator=gen).half().to(device)
                    for _, _, _, layer in column:
                        layer(x)
                    stream.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=stream):
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
                        samples.append(e0.elapsed_time(e1) * 1e3 / len(column))
                    us = statistics.median(samples)
                    gbs = weight_bytes(n, k) / us / 1e3
                    out.append({"proj": name, "N": n, "K": k, "M": m, "us": round(us, 2),
                                "kernel": layer.execution_info(x)["implementation"],
                                "weight_GBps": round(gbs, 1), "frac_of_measured_hbm": round(gbs / hbm_peak, 3),
                                "TFLOPS": round(2.0 * m * n * k / us / 1e6, 2)})
    out.sort(key=lambda r: ([s[0] for s in spec["shapes"]].index(r["proj"]), r["M"]))
    return out


def warm_protocol(stream, device):
    """The reference's own published protocol (benchmarks/bench_hgemm.py:18-45, bench_qwen3_gemm.py:65-83): W and x
    ~ N(0,1) FP16 seeded m+n+k, repeated inputs (weights stay in L2), 8 calls per CUDA graph, median of 21
    replays, microseconds per call - the rows comparable with the reference's RTX 5080 table."""
    import dandan_ops_b200 as ops

    rows = []
    shapes = [("qkv_fused", 4096, 1024), ("o_proj", 1024, 2048), ("gate_up_fused", 6144, 1024), ("down_proj", 1024, 3072)]
    with torch.cuda.stream(stream):
        for name, n, k in shapes:
            for m in (1, 8, 512):
                g = torch.Generator().manual_seed(m + n + k)
                x = torch.randn(m, k, generator=g).half().to(device)
                layer = ops.QuantizedLinear.from_float(torch.randn(n, k, generator=g).half().to(device), group_size=64)
                for _ in range(3):
                    layer(x)
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for _ in range(8):
                        layer(x)
                samples = []
                for _ in range(21):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(stream)
                    graph.replay()
                    e1.record(stream)
                    stream.synchronize()
                    samples.append(e0.elapsed_time(e1) * 1e3 / 8)
                rows.append({"proj": name, "M": m, "N": n, "K": k, "median_us": round(statistics.median(samples), 2),
                             "kernel": layer.execution_info(x)["implementation"]})
    return {"protocol": "repeated inputs (L2-warm), 8 calls per CUDA graph, median of 21 replays, W and x ~ N(0,1) seeded m+n+k",
            "rows": rows}


# ----------------------------------------------------------------------------------------------
# CPU baseline / reference arm: the reference's CPU route on the host cores
# ----------------------------------------------------------------------------------------------
def import_reference():
    """The reference package, if the environment variable B2_REFERENCE_ROOT names a checkout of it; else None."""
    for root in (os.environ.get("B2_REFERENCE_ROOT"),):
        if root and (Path(root) / "dandan_ops" / "quantized_linear.py").is_file():
            sys.path.insert(0, root)
            try:
                import dandan_ops
                return dandan_ops
            except Exception:
                sys.path.remove(root)
    return None


def cpu_states(spec, shapes, reference):
    """Per shape a callable x -> y that runs the reference's CPU route on seeded weights."""
    from oracle import w4a16_oracle as oracle

    runs = []
    for i, (_, n, k) in enumerate(shapes):
        gen = torch.Generator().manual_seed(spec["seed"] + i)
        w = (torch.randn(n, k, generator=gen) * spec["sigma"]).half()
        if reference is not None:
            layer = reference.QuantizedLinear.from_float(w, group_size=64)
            runs.append(layer)
        else:
            codes, step, zero = oracle.quantize(w.numpy())
            words, step, zero = torch.from_numpy(oracle.pack(codes)), torch.from_numpy(step), torch.from_numpy(zero)
            runs.append(lambda x, a=words, b=step, c=zero, kk=k: oracle.torch_forward(x, a, b, c, kk))
    return runs


def cpu_sample(spec):
    shapes = spec["shapes"]
    if max(n * k for _, n, k in shapes) > 200e6:      # bound the sample: eighth-height slices of huge layers
        shapes = [(name, n // 8, k) for name, n, k in shapes]
    return shapes


def cpu_pass(spec, shapes, runs, xs):
    covered = 0.0
    for (name, n, k), run in zip(shapes, runs):
        for m in spec["ms"]:
            run(xs[(m, k)])
            covered += weight_bytes(n, k)
    return covered


def cpu_arm(spec, passes=None, seconds=None, warmup=1):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    reference = import_reference()
    shapes = cpu_sample(spec)
    runs = cpu_states(spec, shapes, reference)
    gen = torch.Generator().manual_seed(spec["seed"] + 5)
    xs = {(m, k): torch.randn(m, k, generator=gen).half() for m in spec["ms"] for k in sorted({k for _, _, k in shapes})}
    for _ in range(max(1, warmup)):
        cpu_pass(spec, shapes, runs, xs)
    covered, t0, done = 0.0, time.perf_counter(), 0
    while (passes is not None and done < passes) or (passes is None and (done < 1 or (time.perf_counter() - t0 < seconds and done < 50))):
        covered += cpu_pass(spec, shapes, runs, xs)
        done += 1
    elapsed = time.perf_counter() - t0
    kind = "reference" if reference is not None else "port"
    what = ("the reference package's QuantizedLinear, CPU route" if reference is not None else
            "torch FP32 matmul restatement of the reference CPU route")
    return {"value": round(covered / elapsed / 1e9, 4), "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"{done} passes over one layer's projections {[f'{n}x{k}' for _, n, k in shapes]} "
                      f"at M={spec['ms']} ({elapsed:.1f} s, {what})"}, elapsed, done


def cpu_baseline(spec, sample_seconds=15.0):
    return cpu_arm(spec, seconds=sample_seconds)[0]


def run_reference(args, rank, world):
    if rank != 0:
        return
    spec = WORKLOADS[args.workload]
    cpu, elapsed, done = cpu_arm(spec, passes=max(1, args.steps), warmup=max(1, min(args.warmup, 2)))
    print(json.dumps({
        "impl": "reference", "metric": "w4a16_decode_weight_hbm_GBps", "value": cpu["value"], "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(elapsed / done * 1e3, 3), "higher_is_better": True,
        "scaling": "strong" if spec["shard"] else "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": args.workload, "batch_sizes": spec["ms"],
                   "shapes_NxK": [f"{n}x{k}" for _, n, k in cpu_sample(spec)],
                   "note": "each step = a bounded sample of the workload: one layer's projections (eighth-height row slices of "
                           "the 70B-class layers) at every decode batch size, all host threads"},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="llama3-70b-mlp")
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--no-gather", action="store_true", help="sharded workload at N > 1: leave the output slices on their ranks")
    ap.add_argument("--separate-gather", action="store_true",
                    help="sharded workload at N > 1: projection and gather as two launches per linear instead of one")
    ap.add_argument("--no-detail", action="store_true", help="skip the per-shape tables")
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
