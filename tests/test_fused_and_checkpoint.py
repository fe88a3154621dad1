"""Fused projection sets (one N-concatenated launch) and checkpoint tooling.

CPU tests cover the state handling; the GPU tests compare with the separate layers and with a
fresh repack."""
import numpy as np
import pytest
import torch

import dandan_ops_b200 as ops
from dandan_ops_b200 import _native, checkpoint
from dandan_ops_b200.fused import FusedProjections, GateUpSilu, RmsNormLinear, concat_layers, fuse_named_projections, pair_order


def _layer(n, k, seed, bias=False, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, k, generator=g) * 0.03).half().to(device)
    b = torch.randn(n, generator=g).half().to(device) if bias else None
    return ops.QuantizedLinear.from_float(w, b)


def test_concat_state_is_the_rows_side_by_side():
    q, k, v = _layer(48, 200, 1), _layer(16, 200, 2), _layer(17, 200, 3)
    fused = FusedProjections([q, k, v], names=["q", "k", "v"])
    assert fused.out_features == 81 and fused.split_sizes == [48, 16, 17]
    assert torch.equal(fused.op.packed_weight[48:64], k.packed_weight)
    assert torch.equal(fused.op.scales[64:], v.scales) and torch.equal(fused.op.zeros[:48], q.zeros)
    back = fused.unfuse()
    for a, b in zip(back, (q, k, v)):
        assert a.bias is None
        for key in ("packed_weight", "scales", "zeros"):
            assert torch.equal(getattr(a, key), getattr(b, key))
        assert a.get_extra_state() == b.get_extra_state()


def test_concat_bias_and_errors():
    a, b = _layer(8, 64, 1, bias=True), _layer(8, 64, 2)
    both = concat_layers([a, b])
    assert torch.equal(both.bias[:8], a.bias) and torch.count_nonzero(both.bias[8:]) == 0
    assert [l.bias is None for l in FusedProjections([a, b]).unfuse()] == [False, True]
    with pytest.raises(ValueError, match="in_features"):
        concat_layers([a, _layer(8, 128, 3)])
    with pytest.raises(TypeError):
        concat_layers([])
    with pytest.raises(ValueError, match="one name"):
        FusedProjections([a, b], names=["only"])


def test_fuse_named_children():
    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj, self.up_proj, self.down_proj = _layer(32, 64, 1), _layer(32, 64, 2), _layer(64, 32, 3)
    block = Block()
    fused = fuse_named_projections(block, ["gate_proj", "up_proj"])
    assert block.gate_proj_up_proj is fused and not hasattr(block, "gate_proj") and hasattr(block, "down_proj")
    assert fused.names == ["gate_proj", "up_proj"] and fused.out_features == 64


def test_pair_order_and_gate_up_state():
    assert pair_order(16).tolist() == [0, 1, 2, 3, 4, 5, 6, 7, 16, 17, 18, 19, 20, 21, 22, 23,
                                       8, 9, 10, 11, 12, 13, 14, 15, 24, 25, 26, 27, 28, 29, 30, 31]
    with pytest.raises(ValueError, match="multiple of 8"):
        pair_order(12)
    gate, up = _layer(24, 130, 1, bias=True), _layer(24, 130, 2)
    fused = GateUpSilu(gate, up)
    assert fused.op.out_features == 48 and fused.out_features == 24
    assert torch.equal(fused.op.packed_weight[8:16], up.packed_weight[0:8])
    assert torch.equal(fused.op.scales[16:24], gate.scales[8:16])
    assert torch.equal(fused.op.bias[:8], gate.bias[:8]) and torch.count_nonzero(fused.op.bias[8:16]) == 0
    g2, u2 = fused.unfuse()
    for a, b in ((g2, gate), (u2, up)):
        for key in ("packed_weight", "scales", "zeros"):
            assert torch.equal(getattr(a, key), getattr(b, key))
    assert torch.equal(g2.bias, gate.bias) and u2.bias is None
    with pytest.raises(ValueError, match="same number of rows"):
        GateUpSilu(gate, _layer(16, 130, 3))
    with pytest.raises(ValueError, match="CUDA FP16"):
        fused(torch.zeros(2, 130))


def test_checkpoint_round_trip_is_unchanged():
    layers = {"model.layers.0.q.": _layer(24, 130, 1, bias=True), "model.layers.0.o.": _layer(40, 64, 2), "": _layer(8, 64, 3)}
    state = checkpoint.export_int4_layers(layers)
    state["model.norm.weight"] = torch.ones(4)
    assert checkpoint.int4_prefixes(state) == sorted(layers)
    loaded = checkpoint.load_int4_layers(state, device="cpu")
    again = checkpoint.export_int4_layers(loaded)
    assert set(again) == set(state) - {"model.norm.weight"}
    for key, value in again.items():
        if isinstance(value, torch.Tensor):
            assert value.dtype == state[key].dtype and torch.equal(value, state[key])
        else:
            assert value == state[key] and value["format_version"] == 2
    broken = dict(state)
    broken["model.layers.0.o._extra_state"] = dict(broken["model.layers.0.o._extra_state"], format_version=3)
    with pytest.raises((ValueError, RuntimeError)):
        checkpoint.load_int4_layers(broken, device="cpu")


def test_image_file_format_and_digest(tmp_path):
    a, b = _layer(24, 130, 1), _layer(24, 130, 2)
    da = checkpoint.state_digest(a.packed_weight, a.scales, a.zeros, a.in_features)
    assert da == checkpoint.state_digest(a.packed_weight.clone(), a.scales.clone(), a.zeros.clone(), 130)
    assert da != checkpoint.state_digest(b.packed_weight, b.scales, b.zeros, b.in_features)
    assert da != checkpoint.state_digest(a.packed_weight, a.scales, a.zeros, 129) and len(da) == 64
    image = np.arange(4672, dtype=np.uint8)
    path = tmp_path / "x.b2img"
    checkpoint.write_image_file(str(path), image, 24, 130)
    assert path.stat().st_size == 64 + 4672 and path.read_bytes()[:8] == b"B2W4IMG1"
    assert np.array_equal(checkpoint.read_image_file(str(path), 24, 130, 4672), image)
    assert checkpoint.read_image_file(str(path), 24, 131, 4672) is None          # another layer's shape
    assert checkpoint.read_image_file(str(path), 24, 130, 4673) is None
    path.write_bytes(path.read_bytes()[:100])                                       # truncated file
    assert checkpoint.read_image_file(str(path), 24, 130, 4672) is None
    assert checkpoint.read_image_file(str(tmp_path / "missing"), 24, 130, 4672) is None


@pytest.mark.gpu
@pytest.mark.parametrize("m", [1, 8, 100, 300])
def test_fused_projections_match_separate_layers(m):
    q, k, v = (_layer(n, 1024, s, bias=(s == 2), device="cuda") for n, s in ((2048, 1), (1000, 2), (24, 3)))
    fused = FusedProjections([q, k, v])
    x = torch.randn(m, 1024, generator=torch.Generator().manual_seed(m)).half().cuda()
    outs = fused(x)
    assert [o.shape[1] for o in outs] == [2048, 1000, 24]
    for got, layer in zip(outs, (q, k, v)):
        want = layer(x)
        torch.testing.assert_close(got, want, atol=2e-3, rtol=2e-3)
        if m <= 16:          # whole-K tile route: the sum order does not depend on N, bits agree
            assert torch.equal(got, want)
    assert _native.status() == 0
    assert fused.execution_info(x)["kernel_plan"]["route"] == q.execution_info(x)["kernel_plan"]["route"]


@pytest.mark.gpu
def test_image_cache_hit_equals_repack(tmp_path):
    cache = checkpoint.ImageCache(tmp_path)
    layer = _layer(300, 1032, 5, device="cuda")
    fresh = layer._native_image().clone()
    assert cache.attach(layer) is False and cache.misses == 1           # built and stored
    twin = ops.QuantizedLinear(layer.packed_weight.clone(), layer.scales.clone(), layer.zeros.clone(), in_features=1032)
    assert cache.attach(twin) is True and cache.hits == 1
    assert torch.equal(twin._native_image(), fresh)
    x = torch.randn(5, 1032).half().cuda()
    assert torch.equal(twin(x), layer(x))
    with pytest.raises(ValueError, match="native image"):
        twin.attach_native_image(fresh[:-16])
    twin.scales.mul_(2)                                                  # state changed: the attached image is dropped
    assert not torch.equal(twin._native_image(), fresh)


@pytest.mark.gpu
def test_image_cache_restart_path_skips_the_repack_and_rejects_damaged_files(tmp_path):
    """`load_layer` on a host state dict: first a miss (repack + store), then a hit that launches no
    repack kernel; a file with a flipped byte fails its CRC and counts as a miss."""
    cache = checkpoint.ImageCache(tmp_path)
    state = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in _layer(300, 1032, 6, bias=True).state_dict().items()}
    first, hit = cache.load_layer(state)
    assert hit is False and cache.misses == 1
    before = _native.launch_count()
    second, hit = cache.load_layer(state)
    assert hit is True and _native.launch_count() == before             # nothing launched: no repack
    assert torch.equal(second._native_image(), first._native_image())
    x = torch.randn(4, 1032).half().cuda()
    assert torch.equal(second(x), first(x)) and second.bias is not None
    (path,) = list(tmp_path.iterdir())
    raw = bytearray(path.read_bytes())
    raw[64 + 1000] ^= 0x10
    path.write_bytes(bytes(raw))
    third, hit = cache.load_layer(state)
    assert hit is False and torch.equal(third._native_image(), first._native_image())    # rebuilt, file rewritten
    assert cache.load_layer(state)[1] is True


@pytest.mark.gpu
@pytest.mark.parametrize("m", [1, 3, 8, 16, 33, 64, 65, 300, 1000])
@pytest.mark.parametrize("rows,k,bias", [(1536, 1024, False), (3072, 1024, True), (1000, 4096, True), (8, 200, False),
                                          (12288, 4096, False), (512, 3072, True)])
def test_gate_up_silu_matches_the_separate_launches(m, rows, k, bias):
    """Fused SiLU(gate)*up against the two projections followed by torch's own FP16 silu and
    multiply on the GPU (the reference's unfused sequence), and against a CPU restatement."""
    gate, up = _layer(rows, k, 7 + rows, bias=bias, device="cuda"), _layer(rows, k, 9 + rows, bias=bias, device="cuda")
    fused = GateUpSilu(gate, up)
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(m + rows)).half().cuda()
    got = fused(x)
    assert got.shape == (m, rows) and _native.status() == 0
    g16, u16 = gate(x), up(x)
    separate = torch.nn.functional.silu(g16) * u16
    # the separate layers may add the K partial sums in another order (other routes, other tile shapes):
    # each sum is within 2e-3 + 2e-3|y| of the other, and the product of two such values within about 1e-2
    torch.testing.assert_close(got, separate, atol=1e-2, rtol=1e-2)
    # on the same FP16 sums the fused arithmetic is the reference's, bit for bit
    pairs = fused.op(x)
    again = _native.silu_mul_pairs(pairs)
    order = pair_order(rows, "cuda")
    gp, upv = pairs[:, :][:, torch.argsort(order)][:, :rows], pairs[:, torch.argsort(order)][:, rows:]
    want = torch.nn.functional.silu(gp) * upv
    mism = (again != want)
    assert float(mism.float().mean()) <= 1e-3           # torch's exp may differ by an ulp before the FP16 rounding
    torch.testing.assert_close(again, want, atol=0, rtol=2e-3)
    assert _native.load().b2_w4a16_silu_mul_is_fused(m, 2 * rows, k) == 1
    assert torch.equal(got, again)                       # in-kernel epilogue == elementwise kernel on the same sums
    cpu = (torch.nn.functional.silu(gp.cpu().float()).half().float() * upv.cpu().float()).half()
    torch.testing.assert_close(again.cpu(), cpu, atol=0, rtol=2e-3)


def test_rmsnorm_linear_argument_checks():
    layer = _layer(16, 64, 1)
    with pytest.raises(ValueError, match="in_features elements"):
        RmsNormLinear(torch.ones(63), layer)
    with pytest.raises(ValueError, match="multiple of 8"):
        RmsNormLinear(torch.ones(60), _layer(16, 60, 2))
    with pytest.raises(ValueError, match="eps"):
        RmsNormLinear(torch.ones(64), layer, eps=-1.0)
    mod = RmsNormLinear(torch.ones(64), layer, eps=1e-6)
    assert mod.norm_weight.dtype == torch.float16 and "norm_weight" in mod.state_dict()
    with pytest.raises(ValueError, match="CUDA FP16"):
        mod(torch.zeros(2, 64, dtype=torch.float16))


def _rms_reference(summed, weight, eps):
    """The reference's CPU formula (dandan_ops/elementwise.py:118-120)."""
    work = summed.float()
    return (work * torch.rsqrt(work.square().mean(-1, keepdim=True) + eps)).to(summed.dtype) * weight


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(1, 4096, 1024), (8, 4096, 1024), (16, 1024, 2048), (5, 1000, 1032),
                                   (8, 24576, 4096), (40, 2048, 1024), (300, 1536, 1024)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_rmsnorm_linear_matches_norm_then_projection(m, n, k, with_residual):
    gen = torch.Generator().manual_seed(m + n + k)
    layer = _layer(n, k, 3 + n, bias=(n == 1000), device="cuda")
    weight = (1.0 + 0.1 * torch.randn(k, generator=gen)).half().cuda()
    x = torch.randn(m, k, generator=gen).half().cuda()
    residual = torch.randn(m, k, generator=gen).half().cuda() if with_residual else None
    mod = RmsNormLinear(weight, layer, eps=1e-6)
    y, summed = mod(x, residual)
    assert _native.status() == 0
    want_sum = (x + residual) if with_residual else x
    assert torch.equal(summed, want_sum)                                   # FP16 add, one rounding
    xn, summed2 = _native.residual_rms_norm(x, residual, weight, 1e-6)
    assert torch.equal(summed2, want_sum)
    assert torch.equal(y, layer(xn))           # one call == norm kernel followed by the projection, bit for bit
    # the norm itself against the reference's CPU formula: the FP32 sum of squares is added in another
    # order, so a normalized value may round to the neighbouring FP16 number now and then
    ref = _rms_reference(want_sum.cpu(), weight.cpu(), 1e-6)
    torch.testing.assert_close(xn.cpu(), ref, atol=1e-6, rtol=2e-3)
    assert float((xn.cpu() != ref).float().mean()) < 5e-3
    expected = ref.double() @ layer.dequantize().half().double().t().cpu()
    if layer.bias is not None:
        expected = (expected.float().half() + layer.bias.half().cpu()).double()
    torch.testing.assert_close(y.cpu().double(), expected, atol=4e-3, rtol=4e-3)
