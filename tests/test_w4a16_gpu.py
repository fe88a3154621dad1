"""Parity of the CUDA engine with the CPU oracle and the committed reference fixtures.

Everything here runs on a GPU through the package's public API, which reaches the
kernels only through the C ABI (ctypes).  Integer/byte results and dequantized weights
must match bit for bit; FP16 outputs must satisfy the reference's own acceptance rule
|y - y_ref| <= 2e-3 + 2e-3*|y_ref| (its CUDA tests use assert_close(atol=2e-3, rtol=2e-3)).
"""
import numpy as np
import pytest
import torch

import cases
import dandan_ops_b200 as ops
from dandan_ops_b200 import _native
from oracle import w4a16_oracle as oracle

pytestmark = pytest.mark.gpu
ARR, META = cases.golden()
ATOL = RTOL = 2e-3


def dev(t):
    return t.cuda() if isinstance(t, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(t)).cuda()


def oracle_y(x, layer):
    return oracle.linear(x.cpu().numpy(), layer.packed_weight.cpu().numpy(), layer.scales.cpu().numpy(),
                         layer.zeros.cpu().numpy(), layer.in_features)


def assert_close_ref(y, y_ref):
    y_ref = torch.as_tensor(y_ref)
    torch.testing.assert_close(y.cpu(), y_ref, atol=ATOL, rtol=RTOL)


def test_library_loaded_and_contract():
    lib = _native.load()
    assert lib.b2_w4a16_contract_version() == 2
    assert torch.ops.dandan_ops.w4a16_contract_version() == 2


@pytest.mark.parametrize("kind,k", [tuple(e) for e in META["edges"]])
def test_edges_state_and_dequant_bit_exact(kind, k):
    tag = f"edge_{kind}_{k}"
    w = dev(ARR[tag + "_w"])
    codes, step, zero = ops.quantize_int4(w)
    assert np.array_equal(codes.cpu().numpy(), ARR[tag + "_codes"])
    assert np.array_equal(step.cpu().numpy().view(np.uint32), ARR[tag + "_step"].view(np.uint32))
    assert np.array_equal(zero.cpu().numpy(), ARR[tag + "_zero"])
    words = ops.pack_int4(codes)
    assert np.array_equal(words.cpu().numpy(), ARR[tag + "_words"])
    assert torch.equal(ops.unpack_int4(words, k), codes)
    deq = ops.dequantize_int4(words, step, zero, k)
    assert np.array_equal(deq.cpu().numpy().view(np.uint32), ARR[tag + "_deq"].view(np.uint32))
    # relayout round trip
    image = _native.repack(words, step, zero, k)
    w2, s2, z2 = _native.unrepack(image, 3, k)
    assert torch.equal(w2, words) and torch.equal(z2, zero)
    assert torch.equal(s2.view(torch.int32), step.view(torch.int32))


def test_nibble_order_known_answer():
    q = torch.tensor([[0, 1, 2, 3, 4, 5, 6, 15, 9]], dtype=torch.uint8, device="cuda")
    words = ops.pack_int4(q)
    assert words.tolist() == [[0xF6543210 - 2**32, 9]]
    assert torch.equal(ops.unpack_int4(words, 9), q)


@pytest.mark.parametrize("case", META["small"], ids=lambda c: c["name"])
def test_small_golden_cases(case):
    name, k = case["name"], case["k"]
    bias = dev(ARR[name + "_bias"]) if case["bias"] else None
    layer = ops.QuantizedLinear.from_float(dev(ARR[name + "_w"]), bias)
    assert np.array_equal(layer.packed_weight.cpu().numpy(), ARR[name + "_words"])
    assert np.array_equal(layer.scales.cpu().numpy().view(np.uint32), ARR[name + "_step"].view(np.uint32))
    assert np.array_equal(layer.zeros.cpu().numpy(), ARR[name + "_zero"])
    y = layer(dev(ARR[name + "_x"]))
    assert y.dtype == torch.float16 and tuple(y.shape) == (case["m"], case["n"])
    assert_close_ref(y, ARR[name + "_y"])


def test_cpu_runnable_config():
    c = META["cases"]["cfg1"]
    w, x = cases.gaussian_case(c["n"], c["k"], c["m"], c["seed"], c["sigma"])
    layer = ops.QuantizedLinear.from_float(w.cuda(), group_size=64)
    assert cases.sha(layer.packed_weight) == c["sha_words"]
    assert cases.sha(layer.scales) == c["sha_step"]
    assert cases.sha(layer.zeros) == c["sha_zero"]
    assert cases.sha(layer.dequantize().half()) == c["sha_deq_fp16"]
    assert layer.storage_bytes == c["storage_bytes"]
    y = layer(x.cuda())
    assert_close_ref(y, ARR["cfg1_y"])
    info = layer.execution_info(x.cuda())
    assert set(c["info"]) <= set(info) and info["implementation"] == "b200_tile"
    assert info["format_version"] == 2 and info["input_copies"] == []
    # run-to-run determinism of the split-K reduction
    assert torch.equal(y, layer(x.cuda()))


@pytest.mark.parametrize("case", META["stress"], ids=lambda c: c["name"])
def test_direct_state_stress_golden(case):
    n, k, m = case["n"], case["k"], case["m"]
    pack = lambda codes: ops.pack_int4(codes.cuda())
    words, step, zero = cases.direct_state(n, k, case["seed"], pack)
    assert cases.sha(words) == case["sha_words"]
    layer = ops.QuantizedLinear(words, step.cuda(), zero.cuda(), in_features=k)
    assert cases.sha(layer.dequantize().half()) == case["sha_deq_fp16"]
    y = layer(cases.stress_x(m, k, case["seed"]).cuda())
    assert_close_ref(y[:, ::case["col_step"]].contiguous(), ARR[case["name"] + "_y"])


TAILS = [(1, 1, 1), (2, 5, 7), (3, 7, 9), (4, 31, 63), (5, 33, 65), (7, 5, 129), (8, 37, 257),
         (1, 2048, 1024), (2, 1024, 3072), (4, 3072, 1024), (8, 1024, 1024),
         (8, 37, 65), (16, 63, 64), (17, 65, 129), (32, 128, 256), (33, 67, 128), (128, 64, 64),
         (129, 127, 257), (256, 128, 512)]


@pytest.mark.parametrize("m,n,k", TAILS)
def test_tails_against_oracle(m, n, k):
    torch.manual_seed(m + n + k)
    layer = ops.QuantizedLinear.from_float(torch.randn(n, k, dtype=torch.float16).cuda())
    x = torch.randn(m, k, dtype=torch.float16).cuda()
    y = layer(x)
    assert_close_ref(y, oracle_y(x, layer))
    # the reference's own oracle formula, evaluated on the GPU from the engine's dequantizer
    expected = (x.float() @ layer.dequantize().half().float().t()).half()
    torch.testing.assert_close(y, expected, atol=ATOL, rtol=RTOL)
    assert layer(x[:0]).shape == (0, n)


@pytest.mark.parametrize("n,k", [(37, 257), (16, 64), (100, 1000), (5, 1), (1000, 1024)])
@pytest.mark.parametrize("kind", ["gauss", "direct", "huge", "tiny"])
def test_kernel_internal_weights_bit_exact(n, k, kind):
    """A one-hot x row reads one weight column: y[m, n] must be exactly fp16(w[n, m])."""
    g = torch.Generator().manual_seed(n * 7 + k)
    if kind == "direct":
        words, step, zero = cases.direct_state(n, k, n + k, lambda c: ops.pack_int4(c.cuda()))
        layer = ops.QuantizedLinear(words, step.cuda(), zero.cuda(), in_features=k)
    else:
        scale = {"gauss": 0.02, "huge": 1e3, "tiny": 1e-7}[kind]
        layer = ops.QuantizedLinear.from_float((torch.randn(n, k, generator=g) * scale).cuda())
    want = oracle.dequantize_fp16(layer.packed_weight.cpu().numpy(), layer.scales.cpu().numpy(),
                                  layer.zeros.cpu().numpy(), k)
    assert np.array_equal(layer.dequantize().half().cpu().numpy().view(np.uint16), want.view(np.uint16))
    eye = torch.eye(k, dtype=torch.float16, device="cuda")
    for rows in (slice(0, min(k, 8)), slice(0, k)):
        y = layer(eye[rows])                       # [rows, n] == W[:, rows]^T
        got = y.t().contiguous().cpu().numpy()
        # value equality: a weight of -0.0 comes out of the sum as +0.0, as in the reference
        assert np.array_equal(got, want[:, rows]) and np.isfinite(got).all()


def test_misaligned_x_nondefault_stream_and_graph():
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        torch.manual_seed(3)
        layer = ops.QuantizedLinear.from_float(torch.randn(37, 256, dtype=torch.float16).cuda(), backend="small")
        x = torch.randn(8 * 256 + 1, dtype=torch.float16).cuda()[1:].view(8, 256)   # 2-byte aligned only
        for _ in range(3):
            layer(x)
        actual = layer(x)
    stream.synchronize()
    assert_close_ref(actual, oracle_y(x, layer))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        output = layer(x)
    x.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.count_nonzero(output) == 0
    with pytest.raises(ValueError, match="M<=8"):
        layer(torch.ones(9, 256, dtype=torch.float16, device="cuda"))
    with pytest.raises(RuntimeError, match="M<=8"):
        torch.ops.dandan_ops.w4a16_small(torch.ones(9, 256, dtype=torch.float16, device="cuda"),
                                         layer.packed_weight, layer.scales, layer.zeros, 64)


def test_graph_replay_without_host_reads(monkeypatch):
    torch.manual_seed(51)
    layer = ops.QuantizedLinear.from_float(torch.randn(67, 129, dtype=torch.float16).cuda())
    one = torch.randn(1, 129, dtype=torch.float16).cuda()
    batch = torch.cat([one, torch.zeros_like(one), one * 2], dim=0)
    expected = oracle_y(one, layer)
    for backend in ("auto", "cuda", "gemv", "tensorcore", "naive"):
        layer.backend = backend
        assert_close_ref(layer(one), expected)
    layer.backend = "reference"
    with pytest.raises(ValueError, match="CUDA FP16"):
        layer(one)
    layer.backend = "cuda"
    eager = layer(batch)
    assert_close_ref(eager[:1], expected)
    graph = torch.cuda.CUDAGraph()

    def forbidden(*a, **kw):
        pytest.fail("forward read a tensor value on the host")

    with monkeypatch.context() as patch:
        patch.setattr(torch.Tensor, "item", forbidden)
        patch.setattr(torch.Tensor, "__bool__", forbidden)
        patch.setattr(torch.Tensor, "tolist", forbidden)
        for _ in range(3):
            layer(batch)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            output = layer(batch)
        for factor in (1.0, -1.0, 0.0):
            batch.copy_(torch.cat([one, torch.zeros_like(one), one * 2], dim=0) * factor)
            graph.replay()
    torch.cuda.synchronize()
    assert torch.count_nonzero(output) == 0
    s = layer.scales.clone()
    layer.cpu().half().cuda().bfloat16()
    assert layer.scales.dtype == torch.float32 and torch.equal(layer.scales, s)
    assert_close_ref(layer(one), expected)     # image rebuilt after the round trip through the CPU


def test_ones_weight_exact_and_ops_surface():
    layer = ops.QuantizedLinear.from_float(torch.ones(67, 129, dtype=torch.float16).cuda())
    for m in (1, 8, 70):
        y = layer(torch.ones(m, 129, dtype=torch.float16, device="cuda"))
        assert torch.equal(y, torch.full_like(y, 129))
    a = torch.randn(8, 129, dtype=torch.float16, device="cuda")
    p, s, z = layer.packed_weight, layer.scales, layer.zeros
    ref = layer(a)
    for name in ("w4a16_tensorcore", "w4a16_gemm", "w4a16_small"):
        assert torch.equal(getattr(torch.ops.dandan_ops, name)(a, p, s, z, 64), ref)
    assert torch.equal(torch.ops.dandan_ops.w4a16_gemv(a[:1].contiguous(), p, s, z, 64), layer(a[:1]))
    with pytest.raises(RuntimeError, match="contiguous"):
        torch.ops.dandan_ops.w4a16_tensorcore(torch.randn(129, 8, dtype=torch.float16, device="cuda").t(), p, s, z, 64)
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        torch.ops.dandan_ops.w4a16_gemv(a[:1].contiguous(), p.cpu(), s, z, 64)
    with pytest.raises(RuntimeError, match="metadata"):
        torch.ops.dandan_ops.w4a16_tensorcore(a, p, s[:, :1].contiguous(), z, 64)
    # functional form with bias: FP16 rounding of the product first, bias added after
    bias = torch.randn(67, device="cuda")
    y = ops.quantized_linear(a, p, s, z, in_features=129, bias=bias)
    assert torch.equal(y, ref + bias.half())


def test_linearity_and_full_size_property():
    """Size-independent properties on a large layer: zero input -> exact zero, a power-of-two
    multiple of x scales y exactly, and columns agree with the GPU-side FP32 matmul of the
    engine's own (bit-exact) FP16 weights."""
    n, k = 6144, 4096
    g = torch.Generator().manual_seed(2000)
    layer = ops.QuantizedLinear.from_float((torch.randn(n, k, generator=g) * 0.02).half().cuda())
    x = torch.randn(16, k, generator=g).half().cuda()
    y = layer(x)
    assert torch.count_nonzero(layer(torch.zeros_like(x))) == 0
    normal = y.abs() >= 2.0 ** -13          # doubling is exact only above the FP16 subnormal range
    assert torch.equal(layer(x * 2)[normal], (y * 2)[normal])
    w16 = layer.dequantize().half()
    expected = (x.double() @ w16.double().t())
    assert (y.double() - expected).abs().max() <= 2e-3 + 2e-3 * expected.abs().max()
    for m in (1, 2, 4, 8):
        assert (layer(x[:m]).double() - expected[:m]).abs().max() <= 4e-3


# ------------------------------------------------------------------------------------------
# tensor-memory GEMM route (M > 64 rows of x)
# ------------------------------------------------------------------------------------------
GEMM_SHAPES = [(65, 5, 8), (100, 1000, 1024), (128, 128, 64), (129, 127, 264), (256, 128, 512), (300, 12289, 1024),
               (512, 192, 1024), (1000, 4096, 3072), (2048, 1024, 4096)]


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
def test_tcgen05_route_against_oracle_formula(m, n, k):
    g = torch.Generator().manual_seed(m + n + k)
    layer = ops.QuantizedLinear.from_float((torch.randn(n, k, generator=g) * 0.05).half().cuda())
    x = torch.randn(m, k, generator=g).half().cuda()
    assert layer.execution_info(x)["implementation"] == "b200_tcgen05"
    y = layer(x)
    forced = _native.linear(x, layer._native_image(), n, k, route=_native.ROUTE_TCGEN05)
    assert torch.equal(y, forced)
    assert _native.status() == 0
    expected = (x.double() @ layer.dequantize().half().double().t())
    err = (y.double() - expected).abs()
    assert bool((err <= ATOL + RTOL * expected.abs()).all())
    # both kernel families must agree within the same tolerance
    stream = _native.linear(x, layer._native_image(), n, k, route=_native.ROUTE_STREAM)
    torch.testing.assert_close(y, stream, atol=ATOL, rtol=RTOL)
    if m * n <= 400000:
        assert_close_ref(y, oracle_y(x, layer))


@pytest.mark.parametrize("n,k", [(37, 264), (1000, 1024), (130, 128)])
def test_tcgen05_internal_weights_bit_exact(n, k):
    """One-hot rows of x through the tensor-memory GEMM return the FP16 weights exactly."""
    words, step, zero = cases.direct_state(n, k, n + 3 * k, lambda c: ops.pack_int4(c.cuda()))
    for layer in (ops.QuantizedLinear(words, step.cuda(), zero.cuda(), in_features=k),
                  ops.QuantizedLinear.from_float((torch.randn(n, k) * 0.02).cuda())):
        want = oracle.dequantize_fp16(layer.packed_weight.cpu().numpy(), layer.scales.cpu().numpy(),
                                      layer.zeros.cpu().numpy(), k)
        eye = torch.eye(k, dtype=torch.float16, device="cuda")
        y = _native.linear(eye, layer._native_image(), n, k, route=_native.ROUTE_TCGEN05)
        got = y.t().contiguous().cpu().numpy()
        assert np.array_equal(got, want) and np.isfinite(got).all()


@pytest.fixture
def gemm_shape():
    """Forces a tile shape of the tensor-memory GEMM for one test and restores the cost model."""
    yield _native.set_gemm_shape
    _native.set_gemm_shape("auto")


@pytest.mark.parametrize("shape", ["128x128", "256x128", "256x192", "pair256", "pair192"])
@pytest.mark.parametrize("m,n,k", [(65, 5, 8), (129, 127, 264), (300, 1000, 1024), (200, 12289, 1032), (1000, 1536, 4096)])
def test_tcgen05_every_tile_shape(gemm_shape, shape, m, n, k):
    """Each tile shape (single-CTA and two-SM pair kernels) on ragged sizes: tails in M, N and K."""
    g = torch.Generator().manual_seed(m * 7 + n + k)
    layer = ops.QuantizedLinear.from_float((torch.randn(n, k, generator=g) * 0.05).half().cuda())
    x = torch.randn(m, k, generator=g).half().cuda()
    bias = torch.randn(n, generator=g).half().cuda()
    gemm_shape(shape)
    y = _native.linear(x, layer._native_image(), n, k, route=_native.ROUTE_TCGEN05)
    yb = _native.linear(x, layer._native_image(), n, k, route=_native.ROUTE_TCGEN05, bias=bias)
    assert _native.status() == 0
    expected = (x.double() @ layer.dequantize().half().double().t())
    err = (y.double() - expected).abs()
    assert bool((err <= ATOL + RTOL * expected.abs()).all())
    assert torch.equal(yb, y + bias)                       # FP16 product first, FP16 bias add second
    if m * n <= 400000:
        assert_close_ref(y, oracle_y(x, layer))


@pytest.mark.parametrize("shape", ["pair256", "pair192"])
def test_pair_kernel_internal_weights_bit_exact(gemm_shape, shape):
    """One-hot rows of x through the two-SM kernel (weights via tensor memory) return the FP16
    weights exactly, and a strided output view is honoured."""
    n, k = 300, 520
    words, step, zero = cases.direct_state(n, k, n + 3 * k, lambda c: ops.pack_int4(c.cuda()))
    layer = ops.QuantizedLinear(words, step.cuda(), zero.cuda(), in_features=k)
    want = oracle.dequantize_fp16(layer.packed_weight.cpu().numpy(), layer.scales.cpu().numpy(),
                                  layer.zeros.cpu().numpy(), k)
    gemm_shape(shape)
    eye = torch.eye(k, dtype=torch.float16, device="cuda")
    y = _native.linear(eye, layer._native_image(), n, k, route=_native.ROUTE_TCGEN05)
    got = y.t().contiguous().cpu().numpy()
    assert np.array_equal(got, want) and np.isfinite(got).all()
    assert _native.status() == 0


@pytest.mark.parametrize("shape,splits", [("pair256", 2), ("pair256", 5), ("pair192", 3), ("pair192", 8)])
@pytest.mark.parametrize("m,n,k", [(129, 127, 4104), (300, 1000, 8192), (512, 1536, 5120)])
def test_pair_kernel_k_split(gemm_shape, shape, splits, m, n, k):
    """K split over several CTAs per tile: FP32 partial tiles through the workspace, added in split
    order.  Same tolerance as one CTA per tile, identical bits from call to call, tickets left zero."""
    g = torch.Generator().manual_seed(m + n + k + splits)
    layer = ops.QuantizedLinear.from_float((torch.randn(n, k, generator=g) * 0.05).half().cuda())
    x = torch.randn(m, k, generator=g).half().cuda()
    bias = torch.randn(n, generator=g).half().cuda()
    image = layer._native_image()
    gemm_shape(shape, splits)
    assert _native.plan(m, n, k)["k_splits"] == min(splits, (k + 255) // 256 // 4)
    y = _native.linear(x, image, n, k, route=_native.ROUTE_TCGEN05)
    again = _native.linear(x, image, n, k, route=_native.ROUTE_TCGEN05)
    yb = _native.linear(x, image, n, k, route=_native.ROUTE_TCGEN05, bias=bias)
    assert _native.status() == 0
    assert torch.equal(y, again) and torch.equal(yb, y + bias)
    expected = (x.double() @ layer.dequantize().half().double().t())
    assert bool(((y.double() - expected).abs() <= ATOL + RTOL * expected.abs()).all())
    gemm_shape(shape, 1)
    one = _native.linear(x, image, n, k, route=_native.ROUTE_TCGEN05)
    torch.testing.assert_close(y, one, atol=ATOL, rtol=RTOL)
    ws = list(_native._workspaces.values())[0]
    assert int(ws[:_native.TICKET_BYTES - 4].view(torch.int32).abs().sum()) == 0


def test_tcgen05_unaligned_falls_back_and_graph_replay():
    torch.manual_seed(9)
    layer = ops.QuantizedLinear.from_float(torch.randn(200, 129, dtype=torch.float16).cuda())
    x = torch.randn(100, 129, dtype=torch.float16).cuda()          # K % 8 != 0: streaming kernel
    assert_close_ref(layer(x), oracle_y(x, layer))
    with pytest.raises(RuntimeError, match="tcgen05"):
        _native.linear(x, layer._native_image(), 200, 129, route=_native.ROUTE_TCGEN05)
    layer = ops.QuantizedLinear.from_float(torch.randn(384, 512, dtype=torch.float16).cuda())
    x = torch.randn(300, 512, dtype=torch.float16).cuda()
    expected = oracle_y(x, layer)
    for _ in range(3):
        layer(x)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = layer(x)
    graph.replay()
    torch.cuda.synchronize()
    assert_close_ref(out, expected)
    x.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.count_nonzero(out) == 0


# ------------------------------------------------------------------------------------------
# the three decode/prefill kernel families agree with each other and with the oracle
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("m,n,k", [(1, 1000, 1024), (3, 37, 257), (8, 2048, 1024), (16, 1024, 3072), (5, 12289, 1024),
                                   (16, 4096, 4096), (1, 16, 6912), (9, 100, 264), (5, 1000, 4352), (1, 1184, 2304),
                                   (8, 512, 8192), (16, 256, 4096), (3, 16, 7000)])
def test_tile_and_stream_routes_agree(m, n, k):
    g = torch.Generator().manual_seed(m * 7 + n + k)
    layer = ops.QuantizedLinear.from_float((torch.randn(n, k, generator=g) * 0.03).half().cuda())
    x = torch.randn(m, k, generator=g).half().cuda()
    image = layer._native_image()
    tile = _native.linear(x, image, n, k, route=_native.ROUTE_TILE)
    stream = _native.linear(x, image, n, k, route=_native.ROUTE_STREAM)
    assert _native.status() == 0
    want = oracle_y(x, layer)
    assert_close_ref(tile, want)
    assert_close_ref(stream, want)
    assert torch.equal(tile, _native.linear(x, image, n, k, route=_native.ROUTE_TILE))     # reproducible
    assert torch.equal(stream, _native.linear(x, image, n, k, route=_native.ROUTE_STREAM))
    assert torch.equal(layer(x), tile)                                                   # what AUTO picks here
    eye = torch.eye(k, dtype=torch.float16, device="cuda")[:min(k, 8)]
    w = oracle.dequantize_fp16(layer.packed_weight.cpu().numpy(), layer.scales.cpu().numpy(),
                               layer.zeros.cpu().numpy(), k)
    got = _native.linear(eye, image, n, k, route=_native.ROUTE_TILE).t().contiguous().cpu().numpy()
    assert np.array_equal(got, w[:, :eye.shape[0]])
    tail = torch.eye(k, dtype=torch.float16, device="cuda")[max(0, k - 8):]               # the last columns of K
    got = _native.linear(tail, image, n, k, route=_native.ROUTE_TILE).t().contiguous().cpu().numpy()
    assert np.array_equal(got, w[:, max(0, k - 8):])


def test_route_limits_are_reported():
    layer = ops.QuantizedLinear.from_float(torch.randn(64, 512, dtype=torch.float16).cuda())
    image = layer._native_image()
    with pytest.raises(RuntimeError, match="tile route"):
        _native.linear(torch.zeros(17, 512, dtype=torch.float16, device="cuda"), image, 64, 512, route=_native.ROUTE_TILE)
    big = ops.QuantizedLinear.from_float(torch.randn(16, 40960, dtype=torch.float16).cuda())
    with pytest.raises(RuntimeError, match="tile route"):
        _native.linear(torch.zeros(1, 40960, dtype=torch.float16, device="cuda"), big._native_image(), 16, 40960,
                       route=_native.ROUTE_TILE)
    with pytest.raises(RuntimeError, match="route"):
        _native.linear(torch.zeros(1, 512, dtype=torch.float16, device="cuda"), image, 64, 512, route=9)


@pytest.mark.parametrize("m,n,k", [(1, 1000, 1024), (8, 67, 129), (16, 4096, 1024), (40, 1001, 520), (8, 6144, 4096),
                                   (300, 1000, 1024), (129, 130, 264), (512, 4104, 1024)])
@pytest.mark.parametrize("bias_dtype", [torch.float32, torch.float16])
def test_fused_bias_keeps_the_reference_rounding_order(m, n, k, bias_dtype):
    g = torch.Generator().manual_seed(m + 3 * n + k)
    bias = (torch.randn(n, generator=g) * 3).to(bias_dtype).cuda()
    layer = ops.QuantizedLinear.from_float((torch.randn(n, k, generator=g) * 0.04).half().cuda(), bias)
    x = torch.randn(m, k, generator=g).half().cuda()
    plain = _native.linear(x, layer._native_image(), n, k)            # product only
    y = layer(x)
    assert torch.equal(y, plain + bias.to(torch.float16))             # bit-exact: fp16(product) + fp16(bias)
    assert torch.equal(ops.quantized_linear(x, layer.packed_weight, layer.scales, layer.zeros, in_features=k,
                                            bias=bias), y)
    layer.bias.mul_(2)                                                 # in-place change is picked up
    assert torch.equal(layer(x), plain + (bias * 2).to(torch.float16))


def test_per_token_fast_path_follows_state_changes():
    """The forward fast path (metadata checks skipped while the state is untouched) still follows
    in-place updates of the state and rejects bad inputs with the reference's errors."""
    g = torch.Generator().manual_seed(77)
    a = ops.QuantizedLinear.from_float((torch.randn(4096, 1024, generator=g) * 0.02).half().cuda())
    x = torch.randn(8, 1024, generator=g).half().cuda()
    y0 = a(x).clone()
    for _ in range(3):
        y1 = a(x)
    assert torch.equal(y0, y1) and _native.status() == 0
    with pytest.raises(ValueError):
        a(x.float())                                   # not the CUDA FP16 case: full checks, reference's error
    with pytest.raises(ValueError):
        a(x[:, :512])
    a.scales.mul_(2)                                   # version counter changes: image rebuilt, checks repeated
    y2 = a(x)
    big = y0.abs() >= 2.0 ** -13
    assert torch.equal(y2[big], (y0 * 2)[big])
    a.backend = "gemv"                                 # attribute reassigned: the M == 1 rule applies again
    with pytest.raises(ValueError, match="M=1"):
        a(x)
    a.backend = "auto"
    assert torch.equal(a(x), y2)
