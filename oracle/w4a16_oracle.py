"""CPU oracle for the W4A16 quantized-linear path.  TEST INFRASTRUCTURE ONLY.

This module restates, in numpy, the arithmetic of the reference operator library's
CPU route for its INT4 linear layer.  It exists so that the CUDA engine can be
checked against an independent implementation; nothing in the shipped package
imports it.  Only the test-suite, the smoke entry point and the benchmark's CPU
baseline leg may call into this file.

Parity status: PINNED.  `tests/test_oracle_golden.py` compares every function here
with fixtures produced by running the reference's own Python code
(`tests/golden/make_golden.py` is the generating script) and with the known-answer
vectors the reference's tests hold.

Reference locations restated (paths inside the reference project):
  quantize   dandan_ops/quantization.py:62-82
  pack       dandan_ops/quantization.py:85-103
  unpack     dandan_ops/quantization.py:106-121
  dequantize dandan_ops/quantization.py:124-143
  linear     dandan_ops/quantized_linear.py:73-81  (route "reference")
  residual_rms_norm  dandan_ops/elementwise.py:118-120, 156-161  (route "torch")
  silu_and_mul       dandan_ops/elementwise.py:168-172           (route "torch")

All arithmetic that the reference performs in FP32 is performed here on
np.float32 arrays so that every intermediate is rounded exactly as torch rounds it.
"""
from __future__ import annotations

import numpy as np

GROUP = 64
_F32 = np.float32
_TINY = np.finfo(np.float32).tiny


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def quantize(weight: np.ndarray, group_size: int = GROUP):
    """Asymmetric min/max uint4 quantization of a [N, K] matrix.

    Follows dandan_ops/quantization.py:62-82: the K axis is zero-padded to a whole
    number of groups (the padding takes part in min/max), the range is widened to
    contain zero, the step is `hi/15 - lo/15` (two divisions, then a subtraction),
    clamped to the smallest normal FP32, an all-zero group gets step 1, and both the
    zero point and the codes are rounded half-to-even and clipped to 0..15.
    Returns (codes uint8 [N,K], step float32 [N,G], zero int32 [N,G]).
    """
    w = np.asarray(weight)
    if w.ndim != 2 or 0 in w.shape:
        raise ValueError("weight must be a non-empty [N, K] matrix")
    if not np.isfinite(w.astype(np.float64)).all():
        raise ValueError("weight must be finite")
    n, k = w.shape
    g = _ceil_div(k, group_size)
    grid = np.zeros((n, g * group_size), dtype=_F32)
    grid[:, :k] = w.astype(_F32)
    grid = grid.reshape(n, g, group_size)
    lo = np.minimum(grid.min(axis=2), _F32(0))
    hi = np.maximum(grid.max(axis=2), _F32(0))
    fifteen = _F32(15)
    step = (hi / fifteen - lo / fifteen).astype(_F32)
    step = np.maximum(step, _TINY)
    step = np.where((hi == 0) & (lo == 0), _F32(1), step).astype(_F32)
    with np.errstate(over="ignore"):
        zero_f = np.clip(np.rint((-lo) / step), 0, 15)
        zero = zero_f.astype(np.int32)
        codes = np.rint(grid / step[:, :, None] + zero.astype(_F32)[:, :, None])
    codes = np.clip(codes, 0, 15).astype(np.uint8).reshape(n, g * group_size)
    return np.ascontiguousarray(codes[:, :k]), step, zero


def pack(codes: np.ndarray) -> np.ndarray:
    """Eight 4-bit codes per int32, code j of a word in bits 4j..4j+3.

    Follows dandan_ops/quantization.py:85-103; K is padded with zero codes to a
    multiple of eight and the top code may set the sign bit of the int32.
    """
    c = np.asarray(codes)
    if c.dtype != np.uint8 or c.ndim != 2 or 0 in c.shape:
        raise ValueError("codes must be a non-empty uint8 [N, K] matrix")
    if (c > 15).any():
        raise ValueError("codes must lie in 0..15")
    n, k = c.shape
    words = _ceil_div(k, 8)
    wide = np.zeros((n, words * 8), dtype=np.uint32)
    wide[:, :k] = c
    wide = wide.reshape(n, words, 8)
    shifts = (np.arange(8, dtype=np.uint32) * 4)[None, None, :]
    return (wide << shifts).sum(axis=2, dtype=np.uint32).view(np.int32)


def unpack(words: np.ndarray, k: int | None = None) -> np.ndarray:
    """Inverse of `pack` (dandan_ops/quantization.py:106-121)."""
    p = np.asarray(words)
    if p.dtype != np.int32 or p.ndim != 2 or 0 in p.shape:
        raise ValueError("words must be a non-empty int32 [N, W] matrix")
    u = p.view(np.uint32)
    shifts = (np.arange(8, dtype=np.uint32) * 4)[None, None, :]
    codes = ((u[:, :, None] >> shifts) & 0xF).astype(np.uint8).reshape(p.shape[0], -1)
    if k is None:
        return codes
    if k <= 0 or _ceil_div(k, 8) != p.shape[1]:
        raise ValueError("k does not match the packed width")
    return np.ascontiguousarray(codes[:, :k])


def dequantize(words, step, zero, k: int, group_size: int = GROUP) -> np.ndarray:
    """FP32 weights `(code - zero) * step` (dandan_ops/quantization.py:124-143).

    The subtraction is exact (small integers); the product is one FP32 rounding.
    """
    codes = unpack(words, k).astype(_F32)
    col_group = np.arange(k) // group_size
    z = np.asarray(zero).astype(_F32)[:, col_group]
    s = np.asarray(step, dtype=_F32)[:, col_group]
    with np.errstate(over="ignore", under="ignore", invalid="ignore"):
        return ((codes - z) * s).astype(_F32)


def dequantize_fp16(words, step, zero, k: int, group_size: int = GROUP) -> np.ndarray:
    """The weights the FP16-activation path multiplies by: FP32 result rounded to FP16."""
    with np.errstate(over="ignore"):
        return dequantize(words, step, zero, k, group_size).astype(np.float16)


def linear(x, words, step, zero, k: int, group_size: int = GROUP, bias=None) -> np.ndarray:
    """y = fp16(x32 @ fp32(fp16(W))^T) (+ fp16(bias)), dandan_ops/quantized_linear.py:73-81.

    FP16 activations only (the one dtype the CUDA engine accepts).  Products of two
    FP16 numbers are exact in FP32; the order of the FP32 additions is whatever the
    BLAS behind numpy chooses, which is why output parity is stated with a tolerance
    while weight parity is exact.
    """
    xa = np.asarray(x)
    if xa.dtype != np.float16 or xa.ndim != 2 or xa.shape[1] != k:
        raise ValueError("x must be float16 [M, K]")
    w = dequantize_fp16(words, step, zero, k, group_size).astype(_F32)
    with np.errstate(over="ignore", invalid="ignore"):
        y = (xa.astype(_F32) @ w.T).astype(np.float16)
        if bias is not None:
            y = (y + np.asarray(bias).astype(np.float16)).astype(np.float16)
    return y


def linear_f64(x, words, step, zero, k: int, group_size: int = GROUP) -> np.ndarray:
    """Same product accumulated in float64: an order-independent yard-stick for tests."""
    w = dequantize_fp16(words, step, zero, k, group_size).astype(np.float64)
    return np.asarray(x).astype(np.float64) @ w.T


def within_tolerance(actual, expected, atol: float = 2e-3, rtol: float = 2e-3) -> bool:
    """The reference's acceptance test for every CUDA route: |a-e| <= atol + rtol*|e|."""
    a = np.asarray(actual).astype(np.float64)
    e = np.asarray(expected).astype(np.float64)
    return bool((np.abs(a - e) <= atol + rtol * np.abs(e)).all())


def residual_rms_norm(x, residual, weight, eps: float):
    """(RMSNorm(x + residual) * weight, x + residual) for FP16 inputs, as the reference's CPU
    route computes them (dandan_ops/elementwise.py:156-161 with `_rms_reference`, :118-120): the
    sum is rounded to FP16 first, the mean of squares and the scaling run in FP32, the
    normalized value is rounded to FP16 before the FP16 multiplication by the weight."""
    xa = np.asarray(x, dtype=np.float16)
    summed = xa if residual is None else (xa + np.asarray(residual, dtype=np.float16)).astype(np.float16)
    work = summed.astype(_F32)
    mean_sq = (work * work).mean(axis=-1, keepdims=True, dtype=_F32)
    inverse = (_F32(1) / np.sqrt(mean_sq + _F32(eps))).astype(_F32)
    normed = (work * inverse).astype(np.float16)
    return (normed * np.asarray(weight, dtype=np.float16)).astype(np.float16), summed


def silu_and_mul(gate, up):
    """SiLU(gate) * up on FP16 inputs (dandan_ops/elementwise.py:168-172): the activation is
    evaluated in FP32, rounded to FP16, then multiplied by `up` in FP16."""
    g = np.asarray(gate, dtype=np.float16).astype(_F32)
    with np.errstate(over="ignore"):
        act = (g / (_F32(1) + np.exp(-g))).astype(np.float16)
    return (act * np.asarray(up, dtype=np.float16)).astype(np.float16)


def storage_bytes(n: int, k: int, group_size: int = GROUP) -> int:
    """Bytes of the reference's three state tensors (int32 words, float32 step, int32 zero)."""
    return n * _ceil_div(k, 8) * 4 + 2 * n * _ceil_div(k, group_size) * 4


# --------------------------------------------------------------------------------------
# Timed CPU baseline: the reference's route "reference" uses torch CPU kernels (an FP32
# matmul on all host threads).  The function below performs the same steps with torch so
# that the number printed beside the GPU result uses the same BLAS the reference would.
# --------------------------------------------------------------------------------------
def torch_forward(x, words, step, zero, k: int, group_size: int = GROUP):
    """Torch restatement of dequantize + FP16 rounding + FP32 matmul, for timing on CPU."""
    import torch

    shifts = torch.arange(8, dtype=torch.int32) * 4
    codes = ((words.unsqueeze(-1) >> shifts) & 0xF).reshape(words.shape[0], -1)[:, :k]
    col_group = torch.arange(k) // group_size
    w = (codes.float() - zero[:, col_group].float()) * step[:, col_group]
    w = w.half().float()
    return (x.float() @ w.t()).half()
