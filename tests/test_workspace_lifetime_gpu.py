"""Workspaces and captured graphs: a CUDA graph keeps the raw address of the workspace it was captured
with (ticket counters that must stay zero, split-K partial tiles), so the binding never releases a
workspace that a kernel has seen - a later, larger request retires the old buffer instead of freeing it."""
import pytest
import torch

import dandan_ops_b200 as ops
from dandan_ops_b200 import _native

pytestmark = pytest.mark.gpu


def test_graph_captured_before_the_workspace_grows_still_replays_correctly():
    g = torch.Generator().manual_seed(11)
    small = ops.QuantizedLinear.from_float((torch.randn(8192, 4096, generator=g) * 0.02).half().cuda())   # split-K partials at M = 4
    big = ops.QuantizedLinear.from_float((torch.randn(24576, 4096, generator=g) * 0.02).half().cuda())
    x4 = torch.randn(4, 4096, generator=g).half().cuda()
    x64 = torch.randn(64, 4096, generator=g).half().cuda()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        want = _native.linear(x4, small._native_image(), 8192, 4096, route=_native.ROUTE_STREAM).clone()
        stream.synchronize()
        ws_before = _native._workspaces[(0, stream.cuda_stream)]
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            y = _native.linear(x4, small._native_image(), 8192, 4096, route=_native.ROUTE_STREAM)
        # an eager call on the same stream that needs a much larger workspace
        need_small = _native.load().b2_w4a16_workspace_bytes(4, 8192, 4096)
        need_big = _native.load().b2_w4a16_workspace_bytes(64, 24576, 4096)
        assert need_big > max(need_small, ws_before.numel())
        _native.linear(x64, big._native_image(), 24576, 4096, route=_native.ROUTE_STREAM)
        stream.synchronize()
        ws_after = _native._workspaces[(0, stream.cuda_stream)]
        assert ws_after.data_ptr() != ws_before.data_ptr() and any(b is ws_before for b in _native._retired)
        # fresh allocations must not land on the retired workspace, and must survive the replays untouched
        fillers = [torch.full((ws_before.numel(),), 0x5A, dtype=torch.uint8, device="cuda") for _ in range(4)]
        assert all(f.data_ptr() != ws_before.data_ptr() for f in fillers)
        for _ in range(3):
            y.zero_()
            graph.replay()
            stream.synchronize()
            assert torch.equal(y, want)
        assert all(bool((f == 0x5A).all()) for f in fillers)
        assert _native.status() == 0


def test_private_workspace_gives_a_graph_its_own_buffer():
    g = torch.Generator().manual_seed(12)
    layer = ops.QuantizedLinear.from_float((torch.randn(8192, 4096, generator=g) * 0.02).half().cuda())
    x = torch.randn(4, 4096, generator=g).half().cuda()
    shared = _native.workspace(torch.device("cuda", 0), 1 << 20)
    with _native.private_workspace() as mine:
        y = _native.linear(x, layer._native_image(), 8192, 4096, route=_native.ROUTE_STREAM)
        assert mine.slot[0] is not None and mine.slot[0].data_ptr() != shared.data_ptr()
    assert any(b is mine.slot[0] for b in _native._retired)           # kept alive after the context
    assert torch.equal(y, _native.linear(x, layer._native_image(), 8192, 4096, route=_native.ROUTE_STREAM))
