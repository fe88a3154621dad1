"""`torch.ops.dandan_ops.w4a16_*`: the reference's native operator surface.

The reference registers four CUDA ops plus a contract-version query from C++
(`dandan_ops/csrc/operators.cu:259-278`, `dandan_ops/csrc/hgemm.cu:89-98`).  Callers
and tests invoke them directly with reference-layout tensors, so the same names exist
here.  All four run the one engine of this package; they differ only in the argument
checks the reference ops make (`w4a16_gemv` wants M == 1, `w4a16_small` M <= 8).  The
checks and their messages follow `check_w4a16` (`dandan_ops/csrc/gemm_checks.h:6-30`).
"""
import torch

from . import _native

_INT_MAX = 2**31 - 1
_SCHEMA = "(Tensor x, Tensor packed_w, Tensor scales, Tensor zeros, int group_size) -> Tensor"
_registered = False


def _need(cond, message):
    if not cond:
        raise RuntimeError(message)


def check_w4a16(x, packed, scales, zeros, group_size):
    tensors = (x, packed, scales, zeros)
    _need(all(t.dim() == 2 for t in tensors), "W4A16 tensors must be 2D")
    _need(all(t.is_cuda for t in tensors), "W4A16 expects CUDA tensors")
    _need(all(t.device == x.device for t in tensors), "W4A16 tensors must share a device")
    _need(x.dtype == torch.float16 and packed.dtype == torch.int32 and scales.dtype == torch.float32
          and zeros.dtype == torch.int32, "invalid W4A16 dtypes")
    _need(all(t.is_contiguous() for t in tensors), "W4A16 tensors must be contiguous")
    m, k = x.shape
    n = packed.shape[0]
    _need(k > 0 and n > 0 and k <= _INT_MAX - 64 and n <= _INT_MAX - 64 and m <= _INT_MAX - 128,
          "invalid W4A16 dimensions")
    _need(0 < group_size <= _INT_MAX - k, "invalid group_size")
    _need(x.numel() <= _INT_MAX and m * n <= _INT_MAX and n * k <= _INT_MAX,
          "W4A16 dimensions exceed the kernel index range")
    _need(packed.shape[1] == (k + 7) // 8, "invalid packed weight shape")
    groups = (k + group_size - 1) // group_size
    _need(tuple(scales.shape) == (n, groups) and zeros.shape == scales.shape,
          "invalid W4A16 metadata shape")


def _run(x, packed, scales, zeros, group_size, rule):
    check_w4a16(x, packed, scales, zeros, group_size)
    rule(x, group_size)
    from .quantized_linear import _image_for
    image = _image_for(packed, scales, zeros, x.shape[1])
    return _native.linear(x, image, packed.shape[0], x.shape[1])


def _rule_any(x, group_size):
    _need(group_size == 64, "W4A16 Tensor Core backend requires group_size=64")


def _rule_small(x, group_size):
    _need(group_size == 64 and x.shape[0] <= 8, "W4A16 small requires group_size=64 and M<=8")


def _rule_gemv(x, group_size):
    _need(x.shape[0] == 1, "w4a16_gemv expects x=[1,K]")
    _need(group_size == 64, "this W4A16 engine requires group_size=64")


def _rule_naive(x, group_size):
    _need(group_size == 64, "this W4A16 engine requires group_size=64")


_OPS = {"w4a16_gemv": _rule_gemv, "w4a16_small": _rule_small,
        "w4a16_tensorcore": _rule_any, "w4a16_gemm": _rule_naive}


SHIM_LOADED = False      # True when the ops come from the C++ operator library (lib/dandan_ops_b200_C.so)


def register():
    """Define the ops once per process (no-op if the names already exist).

    The C++ operator library (csrc/torch_shim/shim.cpp, built by `dandan_ops_b200.build.build_shim`) is loaded
    with `torch.ops.load_library`, as the reference loads its `_C` module (dandan_ops/_extension.py:34); it
    registers the same names with TORCH_LIBRARY.  Where that file has not been built, the names are defined
    from Python over the ctypes binding instead - the same C-ABI kernels either way."""
    global _registered, _library, SHIM_LOADED
    if _registered:
        return
    from . import build as _build
    if _build.SHIM_PATH.is_file() and _build.LIB_PATH.is_file():
        try:
            torch.ops.load_library(str(_build.SHIM_PATH))
            SHIM_LOADED = True
            _registered = True
            return
        except OSError:           # stale binary for another torch: fall through to the Python definitions
            pass
    _library = torch.library.Library("dandan_ops", "FRAGMENT")
    for name, rule in _OPS.items():
        _library.define(name + _SCHEMA)
        _library.impl(name, (lambda x, p, s, z, g, _rule=rule: _run(x, p, s, z, g, _rule)), "CUDA")
    _library.define("w4a16_contract_version() -> int")
    _library.impl("w4a16_contract_version", lambda: _native.load().b2_w4a16_contract_version(),
                  "CompositeExplicitAutograd")
    _registered = True
