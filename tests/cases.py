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
