"""The FP16-step dequantization of the decode kernels (B2_FLAG_FP16_STEPS).

For a layer whose steps are all exactly representable in FP16 - checkpoints that store FP16 scales, the
stress sweep's direct states - (code - zero) * step is exact in FP32, so the FP16-only chain (one FP16
subtract or fma, one FP16 multiply per weight pair) must give the SAME weights as the general
mixed-precision chain: outputs with and without the flag are compared bit for bit on the tile and the
streaming kernels, the weights are read back through one-hot rows of x, and the module sets the flag by
itself exactly when the steps qualify.
"""
import pytest
import torch

import cases
import dandan_ops_b200 as ops
from dandan_ops_b200 import _native
from test_configs_gpu import guarded_linear

pytestmark = pytest.mark.gpu


def _direct_layer(n, k, seed):
    words, step, zero = cases.direct_state(n, k, seed, lambda c: ops.pack_int4(c.cuda()).cpu())
    return ops.QuantizedLinear(words.cuda(), step.cuda(), zero.cuda(), in_features=k)


def test_module_sets_the_flag_only_for_fp16_representable_steps():
    fp16 = _native.FLAG_FP16_STEPS
    assert _direct_layer(100, 300, 1)._image_flags & fp16
    g = torch.Generator().manual_seed(2)
    quantized = ops.QuantizedLinear.from_float((torch.randn(64, 256, generator=g) * 0.02).half().cuda())
    assert not quantized._image_flags & fp16                 # hi/15 - lo/15 is an FP32 number
    layer = _direct_layer(100, 300, 3)
    layer.scales.mul_(1.0001)                                # steps change: the image and its flags are rebuilt
    layer._native_image()
    assert not layer._image_flags & fp16


@pytest.mark.parametrize("route", [_native.ROUTE_TILE, _native.ROUTE_STREAM])
@pytest.mark.parametrize("m", [1, 5, 8, 13, 16])
@pytest.mark.parametrize("n,k", [(1000, 1024), (4096, 3072), (12289, 1032), (2048, 8192), (37, 257)])
def test_fp16_step_chain_is_bit_identical_to_the_general_chain(route, m, n, k):
    layer = _direct_layer(n, k, n + k + m)
    image = layer._native_image()
    x = cases.stress_x(m, k, n + k)[:, :k].contiguous().cuda()
    lib = _native.load()
    if route == _native.ROUTE_TILE and _native.plan(m, n, k)["route"] != "b200_tile":
        pytest.skip("the tile route does not take this shape")
    general = guarded_linear(x, image, n, k, route=route)
    fast = _native.linear(x, image, n, k, route=route, flags=_native.FLAG_FP16_STEPS)
    assert torch.equal(fast, general)
    assert lib.b2_w4a16_linear_flags(x.data_ptr(), k, image.data_ptr(), None, fast.data_ptr(), n, m, n, k, None, 0, None, route, 8) != 0
    assert b"unknown flag" in lib.b2_w4a16_last_error()


@pytest.mark.parametrize("route", [_native.ROUTE_TILE, _native.ROUTE_STREAM])
def test_fp16_step_chain_weights_bit_exact(route):
    """One-hot rows of x read single weight columns: y[m, n] must equal fp16(w[n, col[m]]) exactly, outlier steps
    (x50) and every zero point included."""
    n, k = 600, 1024
    layer = _direct_layer(n, k, 77)
    w16 = layer.dequantize().half()
    for base in (0, 496, k - 16):
        cols = torch.arange(base, base + 16)
        x = torch.zeros(16, k, dtype=torch.float16)
        x[torch.arange(16), cols] = 1.0
        y = _native.linear(x.cuda(), layer._native_image(), n, k, route=route, flags=_native.FLAG_FP16_STEPS)
        assert torch.equal(y, w16[:, cols.cuda()].t().contiguous())
    assert torch.equal(layer(x.cuda()), y)                   # the module's forward takes the same path


@pytest.mark.parametrize("m,n,k", [(300, 1000, 1024), (129, 4096, 3072), (2048, 1536, 4096), (700, 12289, 1032)])
def test_pair_gemm_converters_with_fp16_steps_are_bit_identical(m, n, k):
    """The tensor-memory GEMM's converter warps use the same FP16-only chain under the flag."""
    layer = _direct_layer(n, k, 5 * n + k)
    image = layer._native_image()
    x = cases.stress_x(m, k, n)[:, :k].contiguous().cuda()
    general = guarded_linear(x, image, n, k, route=_native.ROUTE_TCGEN05)
    fast = _native.linear(x, image, n, k, route=_native.ROUTE_TCGEN05, flags=_native.FLAG_FP16_STEPS)
    assert torch.equal(fast, general)
    assert torch.equal(layer(x), fast) and _native.status() == 0
