"""INT4 weight format: quantizer, packer, unpacker, dequantizer and state validation.

Same functions, argument meaning, results and error behaviour as the reference's
`dandan_ops/quantization.py`; the bytes they produce are the reference's on-disk
format (unsigned 4-bit codes, eight per int32 with code j in bits 4j..4j+3, one FP32
step and one int32 zero point per output row and group of inputs).

What differs is where the work runs.  Format conversions that touch every weight on
a CUDA tensor go through the native library (`pack_int4`, `dequantize_int4`); the
quantizer itself stays a sequence of individually rounded FP32 torch operations on the
weight's own device, because its result has to match the reference bit for bit.  There
is no CPU dequantizer: the package computes on the GPU only.
"""
import torch

from . import _native

_STATE_FIELDS = (("packed_weight", torch.int32), ("scales", torch.float32), ("zeros", torch.int32))
CUDA_ONLY = "requires CUDA FP16, group_size=64 and forward inference"


def _positive_int(value):
    return isinstance(value, int) and not isinstance(value, bool) and value > 0


def _require_group_size(group_size):
    if not _positive_int(group_size):
        raise ValueError("group_size must be a positive integer")


def validate_int4_state(packed, scales, zeros, in_features, group_size=64, *, values=False):
    """Check dtypes, ranks, shapes and devices of an INT4 state (reference:
    dandan_ops/quantization.py:30-59).  `values=True` additionally scans the steps
    (finite, > 0) and zero points (0..15); that synchronizes and is meant for
    construction and checkpoint loading only, never for the per-token path."""
    _require_group_size(group_size)
    if not _positive_int(in_features):
        raise ValueError("in_features must be a positive integer")
    for tensor, (name, dtype) in zip((packed, scales, zeros), _STATE_FIELDS):
        if not isinstance(tensor, torch.Tensor) or tensor.dtype != dtype:
            raise TypeError(f"{name} must be a {dtype} Tensor")
        if tensor.ndim != 2 or 0 in tensor.shape:
            raise ValueError(f"{name} must be a non-empty 2D tensor")
        if tensor.device.type not in ("cpu", "cuda"):
            raise ValueError(f"{name} must be on CPU or CUDA")
    rows = packed.shape[0]
    if packed.shape[1] != -(-in_features // 8):
        raise ValueError("invalid packed weight shape")
    meta_shape = (rows, -(-in_features // group_size))
    if tuple(scales.shape) != meta_shape or tuple(zeros.shape) != meta_shape:
        raise ValueError("invalid scales or zeros shape")
    if not (packed.device == scales.device == zeros.device):
        raise ValueError("quantization tensors must share a device")
    if values:
        if not bool(torch.logical_and(torch.isfinite(scales), scales > 0).all()):
            raise ValueError("scales must be finite and strictly positive")
        if not bool(torch.logical_and(zeros >= 0, zeros <= 15).all()):
            raise ValueError("zero points must be in [0,15]")


def quantize_int4(weight, group_size=64):
    """Asymmetric min/max uint4 quantization of a [N, K] FP16/FP32 weight.

    Returns (codes uint8 [N,K], steps float32 [N,G], zero points int32 [N,G]).  The
    operation order reproduces dandan_ops/quantization.py:62-82 exactly: K is
    zero-padded to whole groups, the range is widened to contain 0, the step is
    `hi/15 - lo/15` (dividing first keeps finite inputs finite), clamped to the smallest
    normal FP32, an all-zero group uses step 1, and rounding is half-to-even.
    """
    if not isinstance(weight, torch.Tensor):
        raise TypeError("weight must be a Tensor")
    if weight.ndim != 2 or 0 in weight.shape:
        raise ValueError("weight must be a non-empty [N, K] tensor")
    if weight.dtype not in (torch.float16, torch.float32):
        raise TypeError("weight must be float16 or float32")
    if weight.device.type not in ("cpu", "cuda"):
        raise ValueError("weight must be on CPU or CUDA")
    if not bool(torch.isfinite(weight).all()):
        raise ValueError("weight must contain only finite values")
    _require_group_size(group_size)
    rows, k = weight.shape
    groups = -(-k // group_size)
    span = groups * group_size
    grid = weight.detach().to(torch.float32)
    if span != k:
        grid = torch.nn.functional.pad(grid, (0, span - k))
    grid = grid.view(rows, groups, group_size)
    lo = grid.amin(dim=2).clamp_max(0.0)
    hi = grid.amax(dim=2).clamp_min(0.0)
    # Divide by a tensor, not a Python scalar: CUDA tensors divided by a scalar are
    # multiplied by its reciprocal, which is not the IEEE quotient the CPU path produces.
    fifteen = torch.full_like(hi, 15.0)
    step = hi / fifteen - lo / fifteen
    step = step.clamp_min(torch.finfo(torch.float32).tiny)
    step = torch.where(torch.logical_and(hi == 0, lo == 0), torch.ones_like(step), step)
    zero = (-lo / step).round().clamp(0, 15).to(torch.int32)
    codes = (grid / step[:, :, None] + zero[:, :, None]).round().clamp(0, 15).to(torch.uint8)
    codes = codes.view(rows, span)[:, :k].contiguous()
    return codes, step.to(torch.float32).contiguous(), zero.contiguous()


def pack_int4(qweight):
    """uint8 codes [N,K] in 0..15 -> int32 [N, ceil(K/8)], low nibble first
    (dandan_ops/quantization.py:85-103).  CUDA tensors are packed by the native kernel."""
    if not isinstance(qweight, torch.Tensor):
        raise TypeError("qweight must be a Tensor")
    if qweight.ndim != 2 or 0 in qweight.shape:
        raise ValueError("qweight must be a non-empty 2D tensor")
    if qweight.dtype != torch.uint8:
        raise TypeError("qweight must be uint8")
    if bool((qweight > 15).any()):
        raise ValueError("qweight values must be in [0, 15]")
    if qweight.is_cuda:
        return _native.pack(qweight.contiguous())
    rows, k = qweight.shape
    words = -(-k // 8)
    wide = torch.zeros((rows, words * 8), dtype=torch.int64)
    wide[:, :k] = qweight
    shifts = torch.arange(0, 32, 4, dtype=torch.int64)
    merged = (wide.view(rows, words, 8) << shifts).sum(dim=2)
    return merged.to(torch.int32)      # wraps: bit 31 becomes the sign


def unpack_int4(packed, original_k=None):
    """Inverse of pack_int4 (dandan_ops/quantization.py:106-121)."""
    if not isinstance(packed, torch.Tensor):
        raise TypeError("packed must be a Tensor")
    if packed.ndim != 2 or 0 in packed.shape:
        raise ValueError("packed must be a non-empty 2D tensor")
    if packed.dtype != torch.int32:
        raise TypeError("packed must be int32")
    shifts = torch.arange(0, 32, 4, dtype=torch.int32, device=packed.device)
    codes = ((packed.unsqueeze(-1) >> shifts) & 0xF).to(torch.uint8).reshape(packed.shape[0], -1)
    if original_k is None:
        return codes
    if not _positive_int(original_k) or -(-original_k // 8) != packed.shape[1]:
        raise ValueError("invalid original_k")
    return codes[:, :original_k]


def dequantize_int4(packed, scales, zeros, original_k, group_size=64):
    """FP32 weights `(code - zero) * step`, bit-identical to
    dandan_ops/quantization.py:124-143, computed by the native dequantizer on the GPU.
    CUDA tensors with group_size 64 only."""
    validate_int4_state(packed, scales, zeros, original_k, group_size)
    if not packed.is_cuda or group_size != 64:
        raise ValueError("dequantize_int4 " + CUDA_ONLY.replace(" FP16", ""))
    image = _native.repack(packed.contiguous(), scales.contiguous(), zeros.contiguous(), original_k)
    return _native.dequantize(image, packed.shape[0], original_k)
