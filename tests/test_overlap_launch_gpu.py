"""B2_FLAG_OVERLAP_LAUNCH: the decode kernels launched as programmatic dependents of the previous kernel
of the stream.  Its CTAs may start while that kernel drains, but they read x, bias and the workspace only after
it has completed - so a chain in which every call consumes the previous call's output must give the same bits
with and without the flag, eagerly and replayed from a CUDA graph."""
import pytest
import torch

from dandan_ops_b200 import _native
from dandan_ops_b200.quantized_linear import QuantizedLinear

pytestmark = pytest.mark.gpu
STREAM = _native.ROUTE_STREAM


def _layers(n, k, count, seed):
    g = torch.Generator().manual_seed(seed)
    return [QuantizedLinear.from_float((torch.randn(n, k, generator=g) * 0.02).cuda(), torch.randn(n, generator=g).cuda())
            for _ in range(count)]


def _chain(layers, x, flags, outs, route=STREAM):
    """x -> layer 0 -> layer 1 -> ...: every call's x is the previous call's y (square layers)."""
    cur = x
    for layer, out in zip(layers, outs):
        _native.linear(cur, layer._native_image(), layer.out_features, layer.in_features, route=route, out=out,
                       bias=layer._bias_fp16(), flags=flags)
        cur = out
    return cur


@pytest.mark.parametrize("route", [STREAM, _native.ROUTE_TILE, _native.ROUTE_AUTO])
@pytest.mark.parametrize("m", [1, 8, 16, 40])
@pytest.mark.parametrize("n", [1024, 2048, 4096])
def test_dependent_chain_matches_the_serial_chain(m, n, route):
    if route == _native.ROUTE_TILE and m > 16:
        pytest.skip("the tile route takes at most 16 rows")
    layers = _layers(n, n, 6, 100 + m + n)
    x = torch.randn(m, n, generator=torch.Generator().manual_seed(m)).half().cuda()
    plain = [torch.empty(m, n, dtype=torch.float16, device="cuda") for _ in layers]
    over = [torch.empty(m, n, dtype=torch.float16, device="cuda") for _ in layers]
    _chain(layers, x, 0, plain, route)
    for _ in range(3):
        for t in over:
            t.fill_(float("nan"))
        _chain(layers, x, _native.FLAG_OVERLAP_LAUNCH, over, route)
        torch.cuda.synchronize()
        for a, b in zip(plain, over):
            assert torch.equal(a, b)
    assert _native.status() == 0


@pytest.mark.parametrize("route,n", [(STREAM, 4096), (_native.ROUTE_TILE, 1024)])
def test_graph_replay_of_a_dependent_chain(route, n):
    m = 8
    layers = _layers(n, n, 5, 7)
    x = torch.randn(m, n, generator=torch.Generator().manual_seed(3)).half().cuda()
    plain = [torch.empty(m, n, dtype=torch.float16, device="cuda") for _ in layers]
    over = [torch.empty(m, n, dtype=torch.float16, device="cuda") for _ in layers]
    _chain(layers, x, 0, plain, route)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        _chain(layers, x, _native.FLAG_OVERLAP_LAUNCH, over, route)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with _native.private_workspace(), torch.cuda.graph(graph, stream=stream):
            _chain(layers, x, _native.FLAG_OVERLAP_LAUNCH, over, route)
        for _ in range(4):
            for t in over:
                t.fill_(float("nan"))
            graph.replay()
            stream.synchronize()
            for a, b in zip(plain, over):
                assert torch.equal(a, b)


def test_module_forward_uses_the_flag_on_every_route():
    assert _native.OVERLAP_LAUNCH
    layer = _layers(1024, 1024, 1, 5)[0]
    assert layer._image_flags & _native.FLAG_OVERLAP_LAUNCH
    x = torch.randn(4, 1024, generator=torch.Generator().manual_seed(1)).half().cuda()
    for route in (_native.ROUTE_TILE, _native.ROUTE_STREAM, _native.ROUTE_AUTO):
        want = _native.linear(x, layer._native_image(), 1024, 1024, route=route, bias=layer._bias_fp16())
        got = _native.linear(x, layer._native_image(), 1024, 1024, route=route, bias=layer._bias_fp16(),
                             flags=_native.FLAG_OVERLAP_LAUNCH)
        assert torch.equal(got, want)
    assert torch.equal(layer(x), want)
    with pytest.raises(RuntimeError, match="unknown flag"):
        _native.linear(x, layer._native_image(), 1024, 1024, flags=4)


@pytest.mark.parametrize("m", [1, 8, 40])
def test_fused_gate_up_behind_a_producer_kernel(m):
    """x of the fused gate/up call is written by the call before it; with the flag the result must not change."""
    from dandan_ops_b200.fused import GateUpSilu
    k, inter = 2048, 4096
    g = torch.Generator().manual_seed(17 + m)
    producer = _layers(k, k, 1, 3)[0]
    gate, up = (QuantizedLinear.from_float((torch.randn(inter, k, generator=g) * 0.02).cuda()) for _ in range(2))
    fused = GateUpSilu(gate, up)
    x0 = torch.randn(m, k, generator=g).half().cuda()
    mid = torch.empty(m, k, dtype=torch.float16, device="cuda")
    results = []
    for flags in (0, _native.FLAG_OVERLAP_LAUNCH, _native.FLAG_OVERLAP_LAUNCH):
        mid.fill_(float("nan"))
        _native.linear(x0, producer._native_image(), k, k, out=mid, bias=producer._bias_fp16(), flags=flags)
        results.append(_native.linear_silu_mul(mid, fused.op._native_image(), fused.op.out_features, k,
                                               bias=fused.op._bias_fp16(), flags=flags).clone())
    torch.cuda.synchronize()
    assert torch.equal(results[0], results[1]) and torch.equal(results[0], results[2])
    assert torch.equal(fused(mid), results[0])
