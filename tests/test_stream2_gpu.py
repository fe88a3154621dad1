"""The other forms of the streaming kernel (large layers, M <= 16) and the give-up path of the bounded waits.

Variant 0 / 1 is the shipped kernel (what B2_ROUTE_AUTO runs); 2 / 3 are the 32- / 16-warp double-buffered
forms, 4 the chunk-major two-dimensional split (w4a16_stream2d_kernel) wherever K exceeds the x buffer - all
measured slower or level, kept behind the hook.

The 32-warp form is forced where the size rule would not pick it, so that ragged shapes (N not a
multiple of 16 or 512, K not a multiple of 256 or 8, rows of x in 1..16) reach it; it is compared with
the 16-warp form, with an FP32 product of the bit-exact FP16 weights, and through one-hot rows of x
with the weights themselves.  The give-up path is exercised without hanging anything: a test hook
makes one CTA leave out ONE weight copy while arming its barrier, and shortens the poll limit; the
kernel must return, set bit 0 of the status word, and the next call must be correct again.
"""
import ctypes

import pytest
import torch

import dandan_ops_b200 as ops
from dandan_ops_b200 import _native
from test_configs_gpu import guarded_linear

pytestmark = pytest.mark.gpu


@pytest.fixture
def hooks():
    yield _native.test_hooks
    _native.test_hooks()            # defaults


def _layer(n, k, seed):
    g = torch.Generator().manual_seed(seed)
    return ops.QuantizedLinear.from_float((torch.randn(n, k, generator=g) * 0.02).half().cuda()), g


@pytest.mark.parametrize("variant", [2, 3, 4])
@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(5000, 8192), (12289, 4104), (16384, 2304), (9001, 8198), (4099, 28672)])
def test_forced_32_warp_kernel_on_ragged_shapes(hooks, variant, m, n, k):
    layer, g = _layer(n, k, n + k)
    x = torch.randn(m, k, generator=g).half().cuda()
    image = layer._native_image()
    hooks(stream_variant=variant)
    assert _native.plan(m, n, k)["route"] in ("b200_stream", "b200_tile")
    y2 = guarded_linear(x, image, n, k, route=_native.ROUTE_STREAM)
    again = guarded_linear(x, image, n, k, route=_native.ROUTE_STREAM)
    assert torch.equal(y2, again)                                    # split-K sums do not depend on timing
    hooks(stream_variant=1)
    y1 = guarded_linear(x, image, n, k, route=_native.ROUTE_STREAM)
    ref = x.float() @ layer.dequantize().half().float().t()
    for y in (y1, y2):
        assert float(((y.float() - ref).abs() / (2e-3 + 2e-3 * ref.abs())).max()) <= 1.0


@pytest.mark.parametrize("n,k", [(600, 8192), (1030, 4104)])
@pytest.mark.parametrize("variant", [4, 2])
def test_32_warp_kernel_weights_bit_exact(hooks, variant, n, k):
    """One-hot rows of x read single weight columns: y[m, n] must equal fp16(w[n, col[m]]) exactly
    (variant 4: the two-dimensional split, which 16 rows of x and K = 4104 / 8192 select)."""
    layer, _ = _layer(n, k, 3 * n + k)
    w16 = layer.dequantize().half()
    hooks(stream_variant=variant)
    for base in (0, k - 16):
        cols = torch.arange(base, base + 16)
        x = torch.zeros(16, k, dtype=torch.float16)
        x[torch.arange(16), cols] = 1.0
        y = guarded_linear(x.cuda(), layer._native_image(), n, k, route=_native.ROUTE_STREAM)
        assert torch.equal(y, w16[:, cols.cuda()].t().contiguous())


def _raw_call(lib, x, image, y, ws, n, k, route):
    m = x.shape[0]
    return lib.b2_w4a16_linear_route(x.data_ptr(), k, image.data_ptr(), y.data_ptr(), n, m, n, k, ws.data_ptr(),
                                     ws.numel(), torch.cuda.current_stream().cuda_stream, route)


@pytest.mark.parametrize("route,variant,m,n,k", [(_native.ROUTE_STREAM, 4, 8, 8192, 8192), (_native.ROUTE_STREAM, 2, 8, 8192, 8192), (_native.ROUTE_STREAM, 1, 4, 8192, 4096),
                                                 (_native.ROUTE_STREAM, 1, 40, 2048, 2048), (_native.ROUTE_TILE, 0, 8, 2048, 1024)])
def test_a_wait_that_runs_out_sets_the_status_word_and_returns(hooks, route, variant, m, n, k):
    lib = _native.load()
    layer, g = _layer(n, k, 77 + n)
    image = layer._native_image()
    x = torch.randn(m, k, generator=g).half().cuda()
    hooks(stream_variant=variant)                                      # the plan (and its scratch) depends on the form
    need = int(lib.b2_w4a16_workspace_bytes(m, n, k))
    ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device="cuda")
    y = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    word = ctypes.c_uint(7)
    assert _raw_call(lib, x, image, y, ws, n, k, route) == 0
    assert lib.b2_w4a16_status(ws.data_ptr(), None, ctypes.byref(word)) == 0 and word.value == 0
    good = y.clone()
    # one copy of the first CTA never arrives: its wait must give up after 64 polls, not hang
    hooks(wait_limit=64, skip_copy=0, stream_variant=variant)
    assert _raw_call(lib, x, image, y, ws, n, k, route) == 0
    torch.cuda.synchronize()                                          # returns: nothing spins forever
    assert lib.b2_w4a16_status(ws.data_ptr(), None, ctypes.byref(word)) == 0 and word.value & 1
    # the hook was one-shot; on a re-zeroed workspace the next call is correct bit for bit
    hooks(stream_variant=variant)
    ws.zero_()
    y.zero_()
    assert _raw_call(lib, x, image, y, ws, n, k, route) == 0
    assert lib.b2_w4a16_status(ws.data_ptr(), None, ctypes.byref(word)) == 0 and word.value == 0
    assert torch.equal(y, good)
