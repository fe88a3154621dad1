"""ctypes binding of the C-ABI library (include/b2_w4a16.h) and tensor-level wrappers.

The library is the only compute path of the package: if it cannot be loaded, every
operation that needs it raises ImportError - there is no eager or CPU stand-in.
"""
import ctypes
import os
import threading

import torch

from . import build as _build

OK = 0
ROUTE_AUTO, ROUTE_STREAM, ROUTE_TCGEN05, ROUTE_TILE = 0, 1, 2, 3
ROUTE_NAMES = {ROUTE_STREAM: "b200_stream", ROUTE_TCGEN05: "b200_tcgen05", ROUTE_TILE: "b200_tile"}
GEMM_SHAPES = {"auto": 0, "128x128": 1, "256x128": 2, "256x192": 3, "pair256": 4, "pair192": 5}
STREAM_MAX_M = 64
TICKET_BYTES = 32768

_lib = None
_lock = threading.Lock()

_i64, _vp, _int = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
_SIGNATURES = {
    "b2_w4a16_contract_version": (_int, []),
    "b2_w4a16_last_error": (ctypes.c_char_p, []),
    "b2_w4a16_launch_count": (_i64, []),
    "b2_w4a16_set_gemm_shape": (_int, [_int, _int]),
    "b2_w4a16_test_hooks": (_int, [_int, _int, _int]),
    "b2_w4a16_gather": (_int, [ctypes.POINTER(_vp), ctypes.POINTER(_vp), _i64, _int, _int, _i64, _i64, _i64, _i64, _vp]),
    "b2_w4a16_gather_block_bytes": (_i64, [_int, _i64]),
    "b2_w4a16_linear_gather": (_int, [_vp, _i64, _vp, _vp, ctypes.POINTER(_vp), ctypes.POINTER(_vp), _i64, _int, _int, _i64,
                                      _i64, _i64, _i64, _i64, _vp, _i64, _vp, _int]),
    "b2_w4a16_linear_gather_launches": (_int, [_i64, _i64, _i64, _i64, _int, _int, _i64]),
    "b2_w4a16_gather_status": (_int, [_vp, _vp, ctypes.POINTER(ctypes.c_uint)]),
    "b2_w4a16_gather_wait_limit": (_int, [_i64]),
    "b2_w4a16_noop": (_int, [_vp]),
    "b2_w4a16_native_bytes": (_i64, [_i64, _i64]),
    "b2_w4a16_repack": (_int, [_vp, _vp, _vp, _i64, _i64, _vp, _vp]),
    "b2_w4a16_unrepack": (_int, [_vp, _i64, _i64, _vp, _vp, _vp, _vp]),
    "b2_w4a16_pack": (_int, [_vp, _i64, _i64, _vp, _vp]),
    "b2_w4a16_dequantize": (_int, [_vp, _i64, _i64, _vp, _i64, _vp]),
    "b2_w4a16_dequantize_fp16": (_int, [_vp, _i64, _i64, _vp, _i64, _vp]),
    "b2_w4a16_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "b2_w4a16_status": (_int, [_vp, _vp, ctypes.POINTER(ctypes.c_uint)]),
    "b2_w4a16_linear": (_int, [_vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp]),
    "b2_w4a16_linear_static": (_int, [_vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "b2_w4a16_linear_route": (_int, [_vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp, _int]),
    "b2_w4a16_linear_bias": (_int, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp, _int]),
    "b2_w4a16_linear_flags": (_int, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp, _int, _int]),
    "b2_w4a16_linear_silu_mul": (_int, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp]),
    "b2_w4a16_linear_silu_mul_flags": (_int, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp, _int]),
    "b2_w4a16_silu_mul_is_fused": (_int, [_i64, _i64, _i64]),
    "b2_w4a16_silu_mul_pairs": (_int, [_vp, _i64, _vp, _i64, _i64, _i64, _vp]),
    "b2_w4a16_rmsnorm_linear": (_int, [_vp, _i64, _vp, _i64, _vp, ctypes.c_float, _vp, _i64, _vp, _vp, _vp, _vp, _i64,
                                       _i64, _i64, _i64, _vp, _i64, _vp]),
    "b2_w4a16_residual_rms_norm": (_int, [_vp, _i64, _vp, _i64, _vp, ctypes.c_float, _vp, _i64, _vp, _i64, _i64, _i64, _vp]),
    "b2_w4a16_plan": (_int, [_i64, _i64, _i64, ctypes.POINTER(_int), ctypes.POINTER(_int),
                             ctypes.POINTER(_int), ctypes.POINTER(_int)]),
}
EXPORTS = tuple(_SIGNATURES)


def library_path():
    return _build.LIB_PATH


def load():
    """Load lib/libb2w4a16.so (built by `python -m dandan_ops_b200.build`)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = library_path()
        if not path.is_file():
            raise ImportError(f"{path} is missing: run `python -m dandan_ops_b200.build` "
                              "(the package has no other compute path)")
        lib = ctypes.CDLL(str(path))
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(lib, name)   # AttributeError here = stale binary
            fn.restype, fn.argtypes = restype, argtypes
        if lib.b2_w4a16_contract_version() != 2:
            raise ImportError("incompatible W4A16 contract version in " + str(path))
        _lib = lib
    return _lib


def _check(rc):
    if rc != OK:
        raise RuntimeError("b2_w4a16: " + _lib.b2_w4a16_last_error().decode())


def _stream():
    return torch.cuda.current_stream().cuda_stream


def launch_count():
    return int(load().b2_w4a16_launch_count())


_need_cache = {}


def set_gemm_shape(name="auto", k_splits=0):
    """Force one tile shape of the tensor-memory GEMM (and, for the pair shapes, the number of
    CTAs along K) for every later call (tests, tuning); "auto" / 0 restore the cost model."""
    _check(load().b2_w4a16_set_gemm_shape(GEMM_SHAPES[name], k_splits))
    _need_cache.clear()          # the workspace a problem needs depends on the shape


def test_hooks(wait_limit=0, skip_copy=-1, stream_variant=0):
    """Test hooks of the decode kernels (see include/b2_w4a16.h): poll limit of the bounded waits,
    one weight copy to leave out in the next launch, streaming-kernel form."""
    _check(load().b2_w4a16_test_hooks(wait_limit, skip_copy, stream_variant))
    _need_cache.clear()


def gather_block_bytes(world, mailbox_slice_bytes):
    """Bytes of one rank's flag block + packet mailbox (`b2_w4a16_gather_block_bytes`)."""
    return int(load().b2_w4a16_gather_block_bytes(world, mailbox_slice_bytes))


def gather(y_ptrs, flag_ptrs, mailbox_slice_bytes, rank, m, ld, n_total, slice_cols):
    """`b2_w4a16_gather` on the current stream: `y_ptrs` / `flag_ptrs` are per-rank device addresses
    (ints) of the [m, ld] FP16 buffers and flag blocks as mapped into this process; rank q owns the
    columns [q * slice_cols, min(n_total, (q + 1) * slice_cols))."""
    world = len(y_ptrs)
    ys = (_vp * world)(*y_ptrs)
    fs = (_vp * world)(*flag_ptrs)
    _check(load().b2_w4a16_gather(ys, fs, mailbox_slice_bytes, rank, world, m, ld, n_total, slice_cols, _stream()))


def linear_gather(x, image, k, y_ptrs, flag_ptrs, mailbox_slice_bytes, rank, ld, n_total, slice_cols, bias=None, flags=0):
    """`b2_w4a16_linear_gather` on the current stream: this rank's slice of the projection and the all-gather
    of every rank's slice into the `[m, ld]` buffers at `y_ptrs` - one launch at decode sizes, else the
    projection followed by `b2_w4a16_gather`.  `image` (may be None for a rank without rows) holds the rows
    [rank * slice_cols, ...) of W, `bias` those entries of the FP16 bias."""
    lib = load()
    world = len(y_ptrs)
    m = x.shape[0]
    if m == 0:
        return
    ys = (_vp * world)(*y_ptrs)
    fs = (_vp * world)(*flag_ptrs)
    stream = _stream()
    cols = max(0, min(slice_cols, n_total - rank * slice_cols))
    if image is None or cols == 0:
        _check(lib.b2_w4a16_gather(ys, fs, mailbox_slice_bytes, rank, world, m, ld, n_total, slice_cols, stream))
        return
    device = x.device
    key = (m, cols, k, device.index)
    need = _need_cache.get(key)
    if need is None:
        need = _need_cache[key] = int(lib.b2_w4a16_workspace_bytes(m, cols, k))
    ws = None if _private else _workspaces.get((device.index, stream))
    if ws is None or ws.numel() < need:
        ws = workspace(device, need)
    _check(lib.b2_w4a16_linear_gather(x.data_ptr(), x.stride(0) if m > 1 else k, image.data_ptr(),
                                      bias.data_ptr() if bias is not None else None, ys, fs, mailbox_slice_bytes,
                                      rank, world, m, ld, n_total, slice_cols, k, ws.data_ptr(), ws.numel(), stream, flags))


def linear_gather_launches(m, n_total, slice_cols, k, rank, world, mailbox_slice_bytes):
    """Kernels one `linear_gather` call launches: 1 = projection and gather fused, 2 = projection then gather."""
    return int(load().b2_w4a16_linear_gather_launches(m, n_total, slice_cols, k, rank, world, mailbox_slice_bytes))


def gather_status(flag_ptr):
    word = ctypes.c_uint(0)
    _check(load().b2_w4a16_gather_status(flag_ptr, _stream(), ctypes.byref(word)))
    return int(word.value)


def gather_wait_limit(microseconds=0):
    """How long a gather kernel waits for its peers before it gives up (0 = the default, 5 s)."""
    _check(load().b2_w4a16_gather_wait_limit(microseconds))


def noop():
    """An empty kernel on the current stream (launch floor of a graph node)."""
    _check(load().b2_w4a16_noop(_stream()))


def native_bytes(n, k):
    return int(load().b2_w4a16_native_bytes(n, k))


def repack(packed, scales, zeros, k):
    """Reference-layout CUDA tensors -> native image (uint8 tensor)."""
    lib = load()
    n = packed.shape[0]
    size = lib.b2_w4a16_native_bytes(n, k)
    if size <= 0:
        raise RuntimeError("b2_w4a16: W4A16 dimensions exceed the kernel index range")
    with torch.cuda.device(packed.device):
        image = torch.empty(size, dtype=torch.uint8, device=packed.device)
        _check(lib.b2_w4a16_repack(packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                   n, k, image.data_ptr(), _stream()))
    return image


def image_from_host(host_bytes, device):
    """A native image read back from storage (uint8 CPU tensor) -> uint8 tensor on `device`."""
    if host_bytes.dtype != torch.uint8 or host_bytes.ndim != 1:
        raise ValueError("a native image is a flat uint8 tensor")
    return host_bytes.to(device)


def unrepack(image, n, k):
    lib = load()
    dev = image.device
    words, groups = (k + 7) // 8, (k + 63) // 64
    with torch.cuda.device(dev):
        packed = torch.empty((n, words), dtype=torch.int32, device=dev)
        scales = torch.empty((n, groups), dtype=torch.float32, device=dev)
        zeros = torch.empty((n, groups), dtype=torch.int32, device=dev)
        _check(lib.b2_w4a16_unrepack(image.data_ptr(), n, k, packed.data_ptr(), scales.data_ptr(),
                                     zeros.data_ptr(), _stream()))
    return packed, scales, zeros


def pack(codes):
    lib = load()
    n, k = codes.shape
    with torch.cuda.device(codes.device):
        out = torch.empty((n, (k + 7) // 8), dtype=torch.int32, device=codes.device)
        _check(lib.b2_w4a16_pack(codes.data_ptr(), n, k, out.data_ptr(), _stream()))
    return out


def dequantize(image, n, k, dtype=torch.float32):
    lib = load()
    with torch.cuda.device(image.device):
        out = torch.empty((n, k), dtype=dtype, device=image.device)
        fn = lib.b2_w4a16_dequantize if dtype == torch.float32 else lib.b2_w4a16_dequantize_fp16
        _check(fn(image.data_ptr(), n, k, out.data_ptr(), k, _stream()))
    return out


def plan(m, n, k):
    lib = load()
    route, splits, grid, rows = _int(), _int(), _int(), _int()
    _check(lib.b2_w4a16_plan(m, n, k, ctypes.byref(route), ctypes.byref(splits), ctypes.byref(grid),
                             ctypes.byref(rows)))
    return {"route": ROUTE_NAMES.get(route.value, str(route.value)), "k_splits": splits.value,
            "grid": grid.value, "rows_per_launch": rows.value}


# One scratch buffer per (device, stream): kernels on one stream run in order, so every
# layer launched there can share it.  The ticket prefix is zero on allocation and every
# kernel leaves it zero.
#
# A buffer that has been handed to a kernel is NEVER released: a CUDA graph captured earlier
# holds its raw address (tickets that must stay zero, split-K partial tiles), so when a later
# call needs more room the old buffer moves to `_retired` and stays allocated for the life of
# the process.  Growth is geometric, which bounds the retired total by the size of the live one.
# Graphs that were captured on one stream share that stream's buffer and must not be replayed
# concurrently with each other; capture inside `private_workspace()` to give a graph its own.
_workspaces = {}
_retired = []
_private = []        # stack of [buffer or None, minimum bytes] pushed by private_workspace()


def _grown(device, nbytes, previous):
    size = max(int(nbytes), 1 << 20, 2 * previous.numel() if previous is not None else 0)
    if previous is not None:
        _retired.append(previous)
    return torch.zeros(size, dtype=torch.uint8, device=device)


def workspace(device, nbytes):
    if _private:
        slot = _private[-1]
        if slot[0] is None or slot[0].numel() < nbytes or slot[0].device != device:
            slot[0] = _grown(device, max(int(nbytes), slot[1]), slot[0])
        return slot[0]
    key = (device.index, _stream())
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = _workspaces[key] = _grown(device, nbytes, buf)
    return buf


class private_workspace:
    """Context manager: every call inside uses a workspace of its own instead of the current
    stream's shared one.  Capture a CUDA graph inside it when that graph will be replayed
    concurrently with other work of this library (another stream, another graph): calls that
    overlap on the GPU must not share tickets and partial tiles.  The buffer lives as long as
    the process (a captured graph keeps its address)."""

    def __init__(self, min_bytes=1 << 20):
        self.slot = [None, int(min_bytes)]

    def __enter__(self):
        _private.append(self.slot)
        return self

    def __exit__(self, *exc):
        _private.remove(self.slot)
        if self.slot[0] is not None:
            _retired.append(self.slot[0])
        return False


def status(device=None):
    """Sticky status words of every workspace this process has used on `device`, OR-ed together
    (synchronizes; 0 = every kernel ran to completion)."""
    lib = load()
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    result = 0
    with torch.cuda.device(device):
        buffers = [b for b in list(_workspaces.values()) + _retired + [s[0] for s in _private if s[0] is not None]
                   if b.device == device]
        for ws in buffers:
            word = ctypes.c_uint(0)
            _check(lib.b2_w4a16_status(ws.data_ptr(), _stream(), ctypes.byref(word)))
            result |= int(word.value)
    from . import ops as _ops
    if _ops.SHIM_LOADED:          # the workspaces the C++ operator library handed out
        result |= int(torch.ops.dandan_ops.w4a16_workspace_status())
    return result


STATIC_SCRATCH_BYTES = 8 * 1024 * 1024


def linear_static(x, image, n, k, out):
    """`b2_w4a16_linear_static`: at most 64 rows of x, scratch built into the library, nothing
    allocated - the caller provides `out` ([M, N] FP16).  See include/b2_w4a16.h for the rules
    (first call on a device before any stream capture; overlapping calls race)."""
    lib = load()
    m = x.shape[0]
    with torch.cuda.device(x.device):
        _check(lib.b2_w4a16_linear_static(x.data_ptr(), x.stride(0) if m > 1 else k, image.data_ptr(),
                                          out.data_ptr(), out.stride(0), m, n, k, _stream()))
    return out


FLAG_FP16_STEPS = 1
FLAG_OVERLAP_LAUNCH = 2      # the streaming kernel may start under the previous kernel's tail (see include/b2_w4a16.h)
OVERLAP_LAUNCH = os.environ.get("B2_W4A16_OVERLAP", "1") != "0"


def linear(x, image, n, k, route=ROUTE_AUTO, out=None, bias=None, flags=0):
    """y[M,N] = x[M,K] @ W^T (+ FP16 bias [N]) on the current stream.  x must be CUDA FP16 with unit inner stride.
    `flags`: layer flags of the C ABI (FLAG_FP16_STEPS: every step of the layer is FP16-representable)."""
    lib = _lib if _lib is not None else load()
    m = x.shape[0]
    device = x.device
    if torch.cuda.current_device() != device.index:      # rare: keep the common path free of context switches
        with torch.cuda.device(device):
            return linear(x, image, n, k, route, out, bias, flags)
    y = out if out is not None else torch.empty((m, n), dtype=torch.float16, device=device)
    if m == 0:
        return y
    key = (m, n, k, device.index)
    need = _need_cache.get(key)
    if need is None:
        need = _need_cache[key] = int(lib.b2_w4a16_workspace_bytes(m, n, k))
    stream = torch.cuda.current_stream().cuda_stream
    ws = None if _private else _workspaces.get((device.index, stream))
    if ws is None or ws.numel() < need:
        ws = workspace(device, need)
    rc = lib.b2_w4a16_linear_flags(x.data_ptr(), x.stride(0) if m > 1 else k, image.data_ptr(),
                                   bias.data_ptr() if bias is not None else None, y.data_ptr(),
                                   y.stride(0), m, n, k, ws.data_ptr(), ws.numel(), stream, route, flags)
    if rc != OK:
        _check(rc)
    return y


def linear_silu_mul(x, image, n, k, bias=None, out=None, flags=0):
    """Fused gate/up projection on a pair-ordered image: [M, K] -> [M, N/2] (see include/b2_w4a16.h).
    The epilogue runs inside the decode kernels and the pair GEMM; the few problems that take a
    single-CTA GEMM tile run the projection and then the elementwise pair kernel."""
    lib = load()
    m = x.shape[0]
    device = x.device
    y = out if out is not None else torch.empty((m, n // 2), dtype=torch.float16, device=device)
    if m == 0:
        return y
    with torch.cuda.device(device):
        stream = _stream()
        aligned = x.data_ptr() % 16 == 0 and (m == 1 or x.stride(0) % 8 == 0)
        if not lib.b2_w4a16_silu_mul_is_fused(m, n, k) or (m > STREAM_MAX_M and not aligned and k % 8 == 0):
            full = linear(x, image, n, k, bias=bias, flags=flags)
            _check(lib.b2_w4a16_silu_mul_pairs(full.data_ptr(), full.stride(0), y.data_ptr(), y.stride(0), m, n, stream))
            return y
        ws = workspace(device, int(lib.b2_w4a16_workspace_bytes(m, n, k)))
        _check(lib.b2_w4a16_linear_silu_mul_flags(x.data_ptr(), x.stride(0) if m > 1 else k, image.data_ptr(),
                                                  bias.data_ptr() if bias is not None else None, y.data_ptr(),
                                                  y.stride(0), m, n, k, ws.data_ptr(), ws.numel(), stream, flags))
    return y


def silu_mul_pairs(y_pairs):
    """Elementwise SiLU(gate) * up on a pair-ordered [M, N] FP16 tensor -> [M, N/2]."""
    lib = load()
    m, n = y_pairs.shape
    out = torch.empty((m, n // 2), dtype=torch.float16, device=y_pairs.device)
    with torch.cuda.device(y_pairs.device):
        _check(lib.b2_w4a16_silu_mul_pairs(y_pairs.data_ptr(), y_pairs.stride(0), out.data_ptr(), out.stride(0),
                                           m, n, _stream()))
    return out


def _ptr(t):
    return t.data_ptr() if t is not None else None


def residual_rms_norm(x, residual, weight, eps, want_sum=True):
    """(RMSNorm(x + residual) * weight, fp16(x + residual) or None) for CUDA FP16 [M, K] inputs."""
    lib = load()
    m, k = x.shape
    out = torch.empty((m, k), dtype=torch.float16, device=x.device)
    summed = torch.empty((m, k), dtype=torch.float16, device=x.device) if want_sum else None
    with torch.cuda.device(x.device):
        _check(lib.b2_w4a16_residual_rms_norm(x.data_ptr(), x.stride(0), _ptr(residual),
                                              residual.stride(0) if residual is not None else 0, weight.data_ptr(),
                                              float(eps), _ptr(summed), k, out.data_ptr(), k, m, k, _stream()))
    return out, summed


def rmsnorm_linear(x, residual, weight, eps, image, n, k, bias=None, want_sum=True):
    """y = (RMSNorm(x + residual) * weight) @ W^T (+ bias) and the FP16 sum: the norm kernel, then
    the projection (see include/b2_w4a16.h)."""
    lib = load()
    m = x.shape[0]
    device = x.device
    y = torch.empty((m, n), dtype=torch.float16, device=device)
    summed = torch.empty((m, k), dtype=torch.float16, device=device) if want_sum else None
    if m == 0:
        return y, summed
    with torch.cuda.device(device):
        scratch = torch.empty((m, k), dtype=torch.float16, device=device)
        ws = workspace(device, int(lib.b2_w4a16_workspace_bytes(m, n, k)))
        _check(lib.b2_w4a16_rmsnorm_linear(x.data_ptr(), x.stride(0), _ptr(residual),
                                           residual.stride(0) if residual is not None else 0, weight.data_ptr(),
                                           float(eps), _ptr(summed), k, _ptr(scratch), image.data_ptr(), _ptr(bias),
                                           y.data_ptr(), y.stride(0), m, n, k, ws.data_ptr(), ws.numel(), _stream()))
    return y, summed
