"""Seeded input generators shared by the parity tests, the smoke test and the benchmark.

Every generator uses a CPU `torch.Generator`, so the CPU oracle and the CUDA engine see
identical bits wherever they run.
"""
import hashlib
import json
from pathlib import Path

import numpy as np
import torch

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"


def golden():
    """(arrays, meta) of the fixtures produced by tests/golden/make_golden.py."""
    arrays = np.load(GOLDEN_DIR / "w4a16_golden.npz")
    meta = json.loads((GOLDEN_DIR / "w4a16_golden.json").read_text())
    return arrays, meta


def sha(t):
    a = t.detach().cpu().contiguous().numpy() if isinstance(t, torch.Tensor) else np.ascontiguousarray(t)
    return hashlib.sha256(a.tobytes()).hexdigest()


def gaussian_case(n, k, m, seed, sigma=0.02):
    """W [n,k] ~ N(0, sigma^2) and x [m,k] ~ N(0,1), both FP16, from one generator."""
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, k, generator=g) * sigma).half()
    x = torch.randn(m, k, generator=g).half()
    return w, x


def edge_weight(kind, k):
    """The six weight families of the reference's quantizer edge test, seed = k."""
    torch.manual_seed(k)
    w = torch.randn(3, k)
    if kind == "zero":
        w.zero_()
    elif kind == "constant":
        w.fill_(2.5)
    elif kind == "positive":
        w.abs_()
    elif kind == "negative":
        w = -w.abs()
    elif kind == "tiny":
        w *= 1e-39
    elif kind == "large":
        w *= 1e30
    return w


def direct_state(n, k, seed, pack):
    """INT4 state built without the quantizer (stress sweep): uniform codes and zero
    points, log-normal FP16-representable steps, 1 % of the groups enlarged fifty-fold.
    `pack` is the packing function under test or the oracle's."""
    g = torch.Generator().manual_seed(seed)
    groups = (k + 63) // 64
    codes = torch.randint(0, 16, (n, k), generator=g, dtype=torch.uint8)
    zero = torch.randint(0, 16, (n, groups), generator=g, dtype=torch.int32)
    step = torch.exp(torch.randn(n, groups, generator=g) * 0.5 - 5.0)
    outlier = torch.rand(n, groups, generator=g) < 0.01
    step = torch.where(outlier, step * 50.0, step).half().float()
    return pack(codes), step, zero


def stress_x(m, k, seed):
    g = torch.Generator().manual_seed(seed + 500)
    return torch.randn(m, k, generator=g).half()


# ----------------------------------------------------------------------------------------------
# The benchmark configurations at their own shapes and seeds (fixtures: golden/w4a16_configs.*)
# ----------------------------------------------------------------------------------------------
CONFIGS = {
    "cfg2": {"shapes": [("qkv", 4096, 1024), ("o", 1024, 2048), ("gate_up", 6144, 1024), ("down", 1024, 3072)],
             "ms": [1, 2, 4, 8], "sigma": 0.02, "seed": 1000},
    "cfg3": {"shapes": [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 24576, 4096), ("down", 4096, 12288)],
             "ms": [1, 16, 512, 2048], "sigma": 0.02, "seed": 2000},
    "cfg4": {"shapes": [("gate_up", 57344, 8192), ("down", 8192, 28672)],
             "ms": [1, 8, 256, 4096], "sigma": 0.015, "seed": 3000},
}
STRESS_KS, STRESS_NS, STRESS_MS = (1024, 3072, 8192), (1000, 4096, 12289), (1, 3, 17, 100)


def stress_cases():
    """The 36 (case_idx, n, k, m) combinations of the stress sweep; seed = 4000 + case_idx."""
    out = []
    for k in STRESS_KS:
        for n in STRESS_NS:
            for m in STRESS_MS:
                out.append((len(out), n, k, m))
    return out


def config_inputs(cfg, shape_idx):
    """(W [N,K] FP16, {M: x [M,K] FP16}) of one projection of a benchmark configuration: one CPU
    generator seeded `seed + shape_idx`, W first, then x for every batch size in order."""
    spec = CONFIGS[cfg]
    _, n, k = spec["shapes"][shape_idx]
    g = torch.Generator().manual_seed(spec["seed"] + shape_idx)
    w = (torch.randn(n, k, generator=g) * spec["sigma"]).half()
    xs = {m: torch.randn(m, k, generator=g).half() for m in spec["ms"]}
    return w, xs


def sample_columns(n, count=128, tail=24):
    """Output columns kept in the fixtures: `count` evenly spaced ones plus the last `tail`."""
    cols = set(range(0, n, max(1, n // count))) | set(range(max(0, n - tail), n))
    return sorted(cols)


def sample_rows(m, count=32):
    """Rows of x kept in the fixtures for large batches: evenly spaced plus the last three."""
    if m <= 128:
        return list(range(m))
    return sorted(set(range(0, m, m // count)) | {m - 3, m - 2, m - 1})


def config_golden():
    arrays = np.load(GOLDEN_DIR / "w4a16_configs.npz")
    meta = json.loads((GOLDEN_DIR / "w4a16_configs.json").read_text())
    return arrays, meta


def error_metrics(y, y_ref):
    """max_abs, relative_l2 and the fraction of differing elements, as the reference's benchmark
    reports them (benchmarks/bench_qwen3_gemm.py:100-106), plus the worst ratio to the
    acceptance bound 2e-3 + 2e-3*|y_ref| (<= 1 passes)."""
    a = np.asarray(y, dtype=np.float64)
    b = np.asarray(y_ref, dtype=np.float64)
    diff = np.abs(a - b)
    denom = float(np.linalg.norm(b))
    return {"max_abs": float(diff.max()) if diff.size else 0.0,
            "relative_l2": float(np.linalg.norm(a - b) / denom) if denom > 0 else 0.0,
            "mismatch_fraction": float(np.mean(a != b)) if diff.size else 0.0,
            "bound_ratio": float((diff / (2e-3 + 2e-3 * np.abs(b))).max()) if diff.size else 0.0}


def n2_inputs(idx, m, k):
    """Seeded inputs of the formulas either side of the projection (fixtures n2_*): x, residual,
    norm weight, gate, up - all FP16, one generator seeded 5000 + idx."""
    g = torch.Generator().manual_seed(5000 + idx)
    x = torch.randn(m, k, generator=g).half()
    res = torch.randn(m, k, generator=g).half()
    wn = (1.0 + 0.1 * torch.randn(k, generator=g)).half()
    gate = (torch.randn(m, k, generator=g) * 2).half()
    up = torch.randn(m, k, generator=g).half()
    return x, res, wn, gate, up
