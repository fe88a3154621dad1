"""`b2_w4a16_linear_static`: the entry point for callers that can neither allocate device
memory nor pass a workspace (an operator slot that receives only inputs and outputs, a
runtime with frozen memory planning).  It uses a scratch array compiled into the library.

Called here straight through the C ABI (ctypes) and compared with the regular entry point
`b2_w4a16_linear` on the same inputs, twice in a row so that the second call runs on the
scratch the first one left behind.  This file sorts last on purpose: a run that stops at the
first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

import dandan_ops_b200 as ops
from dandan_ops_b200 import _native
from oracle import w4a16_oracle as oracle

pytestmark = pytest.mark.gpu
ATOL = RTOL = 2e-3          # the tolerance of every output comparison in this suite


def _raw_static(lib, x, image, y, m, n, k):
    return lib.b2_w4a16_linear_static(x.data_ptr(), k, image.data_ptr(), y.data_ptr(), n, m, n, k,
                                      torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("m,n,k", [(1, 4096, 1024), (8, 1024, 3072), (16, 6144, 4096), (3, 1000, 1032), (64, 1024, 2048)])
def test_static_scratch_entry_matches_workspace_entry_twice(m, n, k):
    lib = _native.load()
    g = torch.Generator().manual_seed(m * 31 + n + k)
    layer = ops.QuantizedLinear.from_float((torch.randn(n, k, generator=g) * 0.02).half().cuda())
    image = layer._native_image()
    x1 = torch.randn(m, k, generator=g).half().cuda()
    x2 = torch.randn(m, k, generator=g).half().cuda()
    outs = [torch.empty(m, n, dtype=torch.float16, device="cuda") for _ in range(2)]
    _raw_static(lib, x1, image, outs[0], m, n, k)          # set-up call (looks up the scratch address once)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for x, y in zip((x1, x2), outs):                       # two calls in a row on the shared scratch
        assert _raw_static(lib, x, image, y, m, n, k) == 0, lib.b2_w4a16_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before     # the calls took no device memory
    word = ctypes.c_uint(9)
    assert lib.b2_w4a16_status(None, None, ctypes.byref(word)) == 0 and word.value == 0    # status of the built-in scratch
    words, step, zero = (t.cpu().numpy() for t in (layer.packed_weight, layer.scales, layer.zeros))
    for x, y in zip((x1, x2), outs):                       # and against the CPU oracle directly
        ref = oracle.linear(x.cpu().numpy(), words, step, zero, k)
        assert oracle.within_tolerance(y.cpu().numpy(), ref, ATOL, RTOL)
    for x, y in zip((x1, x2), outs):
        want = _native.linear(x, image, n, k)              # existing entry point, caller-owned workspace
        torch.testing.assert_close(y, want, atol=ATOL, rtol=RTOL)
        same_kernel = _native.linear(x, image, n, k, route=_native.ROUTE_STREAM)
        assert torch.equal(y, same_kernel)                 # same kernel, same plan: identical bits
    assert torch.equal(_native.linear_static(x1, image, n, k, outs[0]),
                       _native.linear(x1, image, n, k, route=_native.ROUTE_STREAM))


def test_static_scratch_entry_rejects_what_it_cannot_hold():
    lib = _native.load()
    layer = ops.QuantizedLinear.from_float(torch.randn(256, 512, dtype=torch.float16).cuda())
    image = layer._native_image()
    x = torch.randn(65, 512, dtype=torch.float16, device="cuda")
    y = torch.empty(65, 256, dtype=torch.float16, device="cuda")
    assert _raw_static(lib, x, image, y, 65, 256, 512) != 0
    assert b"at most 64 rows" in lib.b2_w4a16_last_error()
    # a plan whose partial tiles exceed the built-in scratch is refused with both sizes in the message
    # (the sizes are checked before any pointer is used, so placeholders serve as operands)
    n, k, m = 57344, 8192, 64
    assert lib.b2_w4a16_workspace_bytes(m, n, k) > _native.STATIC_SCRATCH_BYTES
    dummy = torch.empty(16, dtype=torch.uint8, device="cuda")
    rc = lib.b2_w4a16_linear_static(dummy.data_ptr(), k, dummy.data_ptr(), dummy.data_ptr(), n, m, n, k, None)
    assert rc != 0 and str(_native.STATIC_SCRATCH_BYTES).encode() in lib.b2_w4a16_last_error()
    assert _raw_static(lib, x[:0], image, y[:0], 0, 256, 512) == 0      # empty batch: nothing to do
