"""Signed-INT4 / group-128 engine format -> operator format (reference:
dandan_ops/integrations/myvllm.py, tests/test_myvllm_adapter.py).  The engine's own packer is
not available here; a symmetric absmax/7 packer of the documented storage format stands in."""
import numpy as np
import pytest
import torch

import dandan_ops_b200 as ops
from dandan_ops_b200.integrations.myvllm import EngineQuantLinear, convert_signed_int4, install_int4_projections
from oracle import w4a16_oracle as oracle


def signed_pack(w, group=128):
    """Symmetric signed INT4: scale = absmax/7 per group (1 for an all-zero group), codes in
    [-8, 7] as two's-complement nibbles, two per byte, low nibble first, K padded to the group."""
    n, k = w.shape
    groups = -(-k // group)
    grid = torch.zeros((n, groups * group), dtype=torch.float32, device=w.device)
    grid[:, :k] = w.float()
    blocks = grid.view(n, groups, group)
    scale = blocks.abs().amax(dim=2) / 7.0
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    q = (blocks / scale[:, :, None]).round().clamp(-8, 7).to(torch.int16).view(n, -1)
    nib = (q & 0xF).to(torch.uint8)
    return (nib[:, 0::2] | (nib[:, 1::2] << 4)).contiguous(), scale.contiguous(), q[:, :k].float()


@pytest.mark.parametrize("k", [1, 7, 8, 63, 64, 65, 127, 128, 129, 255, 256, 257, 1024])
@pytest.mark.parametrize("kind", ["random", "zero", "constant"])
def test_bridge_preserves_exact_fp32_weight(k, kind):
    torch.manual_seed(k)
    w = torch.randn(7, k)
    if kind == "zero":
        w.zero_()
    if kind == "constant":
        w.fill_(-0.7)
    packed, scale, q = signed_pack(w)
    words, steps, zeros = convert_signed_int4(packed, scale, k)
    assert words.dtype == torch.int32 and steps.dtype == torch.float32 and zeros.dtype == torch.int32
    assert words.shape == (7, (k + 7) // 8) and steps.shape == zeros.shape == (7, (k + 63) // 64)
    assert int(zeros.min()) == int(zeros.max()) == 8
    want = q * scale.repeat_interleave(128, dim=1)[:, :k]            # the engine's own dequantization
    got = oracle.dequantize(words.numpy(), steps.numpy(), zeros.numpy(), k)
    assert np.array_equal(got, want.numpy())


def test_bridge_all_signed_nibbles_and_bad_metadata():
    nibble = torch.arange(16, dtype=torch.uint8).repeat(8).view(1, -1)
    raw = nibble[:, ::2] | (nibble[:, 1::2] << 4)
    words, steps, zeros = convert_signed_int4(raw, torch.ones(1, 1), 128)
    signed = torch.where(nibble >= 8, nibble.short() - 16, nibble.short()).float()
    assert np.array_equal(oracle.dequantize(words.numpy(), steps.numpy(), zeros.numpy(), 128), signed.numpy())
    with pytest.raises(ValueError, match="group"):
        convert_signed_int4(raw, torch.ones(1, 1), 128, 64)
    with pytest.raises(ValueError, match="shape"):
        convert_signed_int4(raw, torch.ones(1, 2), 128)
    with pytest.raises(ValueError, match="positive"):
        convert_signed_int4(raw, torch.zeros(1, 1), 128)
    with pytest.raises(TypeError, match="uint8"):
        convert_signed_int4(raw.int(), torch.ones(1, 1), 128)
    with pytest.raises(TypeError, match="FP32"):
        convert_signed_int4(raw, torch.ones(1, 1).half(), 128)


@pytest.mark.gpu
def test_engine_linear_keeps_leading_dims_and_installs_into_a_model():
    torch.manual_seed(5)

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = torch.nn.Linear(256, 384, bias=False)
            self.o_proj = torch.nn.Linear(384, 256, bias=True)

    class Toy(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.model = torch.nn.Module()
            self.model.layers = torch.nn.ModuleList([Block(), Block()])
            self.lm_head = torch.nn.Linear(256, 100, bias=False)

    toy = Toy().half().cuda()
    reference_w = toy.model.layers[0].q_proj.weight.detach().clone()
    report = install_int4_projections(toy, lambda lin: signed_pack(lin.weight.detach())[:2])
    assert report["replaced_layers"] == ["model.layers.0.q_proj", "model.layers.0.o_proj",
                                         "model.layers.1.q_proj", "model.layers.1.o_proj"]
    assert isinstance(toy.lm_head, torch.nn.Linear) and report["projection_storage_ratio"] > 3
    with pytest.raises(ValueError, match="already quantized"):
        install_int4_projections(toy, lambda lin: signed_pack(lin.weight.detach())[:2])
    layer = toy.model.layers[0].q_proj
    assert isinstance(layer, EngineQuantLinear)
    packed, scale, q = signed_pack(reference_w)
    want_w = (q * scale.repeat_interleave(128, dim=1)[:, :256])
    assert torch.equal(layer.dequantize(), want_w)                    # lossless bridge, exact GPU dequantizer
    x = torch.randn(2, 3, 256, dtype=torch.float16, device="cuda")
    y = layer(x)
    assert y.shape == (2, 3, 384)
    expected = (x.reshape(-1, 256).double() @ want_w.half().double().t()).reshape(2, 3, 384)
    assert bool(((y.double() - expected).abs() <= 2e-3 + 2e-3 * expected.abs()).all())
    with pytest.raises(ValueError, match="CUDA FP16"):
        layer(x.bfloat16())
    o = toy.model.layers[1].o_proj
    assert o.op.bias is not None and o(torch.randn(5, 384, dtype=torch.float16, device="cuda")).shape == (5, 256)


def test_reference_call_shape_with_a_config_object():
    """`install_int4_projections(model, config)` and `EngineQuantLinear(linear, config)`, the reference's
    signatures (dandan_ops/integrations/myvllm.py:54-66, 87): the config is validated with the reference's
    wording; without the external engine on the path the packer must be given, else ImportError."""
    from types import SimpleNamespace

    good = SimpleNamespace(canonical_weight_dtype="int4", activation_dtype="fp16", group_size=128, symmetric=True)
    model = torch.nn.Module()
    model.model = torch.nn.Module()
    model.model.layers = torch.nn.ModuleList([torch.nn.Linear(128, 16, bias=False)])
    for bad in (dict(group_size=64), dict(symmetric=False), dict(activation_dtype="bf16"), dict(canonical_weight_dtype="int8")):
        cfg = SimpleNamespace(**{**vars(good), **bad})
        with pytest.raises(ValueError, match="symmetric INT4, FP16 activation, group_size=128"):
            install_int4_projections(model, cfg)
        with pytest.raises(ValueError, match="symmetric INT4, FP16 activation, group_size=128"):
            EngineQuantLinear(model.model.layers[0], cfg)
    with pytest.raises(ValueError, match="CUDA FP16"):                 # a CPU model is refused before any packing
        install_int4_projections(model, good, packer=lambda lin: signed_pack(lin.weight.detach())[:2])
    with pytest.raises(ValueError, match="CUDA FP16"):
        EngineQuantLinear(model.model.layers[0], good)
    with pytest.raises(TypeError, match="config or a packer"):
        install_int4_projections(model, 3)
    with pytest.raises(TypeError, match="nn.Linear"):
        EngineQuantLinear(torch.zeros(1), good)
    assert getattr(model, "quantization_report", None) is None and isinstance(model.model.layers[0], torch.nn.Linear)


@pytest.mark.gpu
def test_reference_call_shape_on_a_gpu_model():
    from types import SimpleNamespace

    good = SimpleNamespace(canonical_weight_dtype="int4", activation_dtype="fp16", group_size=128, symmetric=True)
    torch.manual_seed(9)
    model = torch.nn.Module()
    model.model = torch.nn.Module()
    model.model.layers = torch.nn.ModuleList([torch.nn.Linear(256, 64, bias=True)])
    model = model.half().cuda()
    with pytest.raises(ImportError, match="mini_engine"):               # the external engine is not installed here
        install_int4_projections(model, good)
    assert isinstance(model.model.layers[0], torch.nn.Linear)           # untouched after the failure
    pack = lambda lin: signed_pack(lin.weight.detach())[:2]            # noqa: E731
    single = EngineQuantLinear(model.model.layers[0], good, pack_linear=pack)
    report = install_int4_projections(model, good, packer=pack)
    assert report["replaced_layers"] == ["model.layers.0"] and report["source_group_size"] == 128
    x = torch.randn(3, 256, dtype=torch.float16, device="cuda")
    assert torch.equal(model.model.layers[0](x), single(x))
