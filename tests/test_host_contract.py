"""CPU tests of the host side: state lifecycle, validation, error wording, C-ABI exports.

These mirror the reference's CPU contract tests (tests/test_quantized_contract.py and
tests/test_dandan_ops_api.py of the reference project) for everything that does not
compute on a device; compute on CPU tensors must fail loudly instead of falling back.
"""
import copy
import ctypes
import io
import re
from pathlib import Path

import numpy as np
import pytest
import torch

import cases
import dandan_ops_b200 as ops
from dandan_ops_b200 import _native, build as b2build
from dandan_ops_b200.quantization import validate_int4_state

ARR, META = cases.golden()
ROOT = Path(__file__).resolve().parent.parent


def test_library_builds_loads_and_exports_every_declared_symbol():
    b2build.build()
    lib = ctypes.CDLL(str(b2build.LIB_PATH))
    header = (ROOT / "include" / "b2_w4a16.h").read_text()
    declared = sorted(set(re.findall(r"\b(b2_w4a16_\w+)\s*\(", header)))
    assert len(declared) >= 14
    for name in declared:
        assert hasattr(lib, name), name
    assert set(_native.EXPORTS) <= set(declared)
    assert _native.load().b2_w4a16_contract_version() == 2
    # pure host arithmetic works without a device
    assert _native.native_bytes(2048, 1024) == 128 * 4 * 2336
    assert _native.native_bytes(16, 256) == 2336 and _native.native_bytes(17, 257) == 4 * 2336
    plan = _native.plan(8, 2048, 1024)
    assert plan["route"] == "b200_tile" and plan["grid"] == 128
    # few row tiles and a long K: a cluster of 2 or 4 CTAs per row tile, each at least 8 half blocks of K
    assert _native.plan(1, 1024, 3072) == {"route": "b200_tile", "k_splits": 2, "grid": 128, "rows_per_launch": 1}
    assert _native.plan(8, 512, 8192) == {"route": "b200_tile", "k_splits": 4, "grid": 128, "rows_per_launch": 8}
    assert _native.plan(16, 1024, 1024)["k_splits"] == 1 and _native.plan(16, 4096, 4096)["k_splits"] == 1
    assert _native.plan(8, 57344, 8192)["route"] == "b200_stream"
    assert _native.plan(32, 2048, 1024)["route"] == "b200_stream"
    assert _native.plan(512, 4096, 4096)["route"] == "b200_tcgen05"
    assert _native.plan(512, 4096, 4097)["route"] == "b200_stream"       # K % 8 != 0
    lib2 = _native.load()
    assert lib2.b2_w4a16_workspace_bytes(8, 2048, 1024) >= 16384
    assert lib2.b2_w4a16_native_bytes(0, 5) == 0
    assert lib2.b2_w4a16_repack(None, None, None, 4, 4, None, None) != 0
    assert b"null" in lib2.b2_w4a16_last_error()


@pytest.mark.parametrize("kind,k", [tuple(e) for e in META["edges"]])
def test_quantize_pack_unpack_match_reference_fixtures(kind, k):
    tag = f"edge_{kind}_{k}"
    codes, step, zero = ops.quantize_int4(torch.from_numpy(ARR[tag + "_w"]))
    assert np.array_equal(codes.numpy(), ARR[tag + "_codes"])
    assert np.array_equal(step.numpy().view(np.uint32), ARR[tag + "_step"].view(np.uint32))
    assert np.array_equal(zero.numpy(), ARR[tag + "_zero"])
    words = ops.pack_int4(codes)
    assert np.array_equal(words.numpy(), ARR[tag + "_words"])
    assert torch.equal(ops.unpack_int4(words, k), codes)
    assert step.dtype == torch.float32 and zero.dtype == torch.int32 and codes.dtype == torch.uint8


def test_cpu_runnable_config_state_matches_reference():
    c = META["cases"]["cfg1"]
    w, _ = cases.gaussian_case(c["n"], c["k"], c["m"], c["seed"], c["sigma"])
    layer = ops.QuantizedLinear.from_float(w, group_size=64)
    assert cases.sha(layer.packed_weight) == c["sha_words"]
    assert cases.sha(layer.scales) == c["sha_step"]
    assert cases.sha(layer.zeros) == c["sha_zero"]
    assert layer.storage_bytes == c["storage_bytes"]
    assert layer.get_extra_state() == META["extra_state"] | {"original_shape": [c["n"], c["k"]]}
    assert list(ops.BACKENDS) == META["backends"] and ops.FORMAT_VERSION == 2


def test_nibble_order_and_shapes():
    q = torch.tensor([[0, 1, 2, 3, 4, 5, 6, 15, 9]], dtype=torch.uint8)
    words = ops.pack_int4(q)
    assert words.tolist() == [[0xF6543210 - 2**32, 9]]
    assert torch.equal(ops.unpack_int4(words, 9), q)
    codes, _, _ = ops.quantize_int4(torch.randn(3, 65))
    assert ops.pack_int4(codes).shape == (3, 9)
    with pytest.raises(ValueError, match="original_k"):
        ops.unpack_int4(words, 17)
    with pytest.raises(ValueError, match=r"\[0, 15\]"):
        ops.pack_int4(torch.full((1, 8), 16, dtype=torch.uint8))
    with pytest.raises(TypeError, match="uint8"):
        ops.pack_int4(torch.zeros(1, 8, dtype=torch.int32))


@pytest.mark.parametrize("bad", [float("nan"), float("inf"), -float("inf")])
def test_reject_nonfinite_weight(bad):
    with pytest.raises(ValueError, match="finite"):
        ops.quantize_int4(torch.tensor([[0.0, bad]]))


@pytest.mark.parametrize("group", [0, -1, True, None, 1.5])
def test_invalid_group(group):
    with pytest.raises(ValueError, match="group_size"):
        ops.QuantizedLinear.from_float(torch.ones(1, 8), group_size=group)


def test_other_group_sizes_keep_their_state_but_cannot_run():
    layer = ops.QuantizedLinear.from_float(torch.randn(4, 96), group_size=32)
    assert layer.scales.shape == (4, 3) and layer.get_extra_state()["group_size"] == 32
    assert layer.execution_info(torch.ones(1, 96).half())["implementation"] == "unavailable"


@pytest.mark.parametrize("field,value,pattern", [
    ("scales", 0.0, "positive"), ("scales", -1.0, "positive"), ("scales", float("inf"), "finite"),
    ("scales", float("nan"), "finite"), ("zeros", 16, "zero points"), ("zeros", -1, "zero points")])
def test_reject_bad_values_at_load(field, value, pattern):
    layer = ops.QuantizedLinear.from_float(torch.ones(3, 65))
    state = copy.deepcopy(layer.state_dict())
    state[field].fill_(value)
    with pytest.raises((ValueError, RuntimeError), match=pattern):
        ops.QuantizedLinear.from_state_dict(state)
    before = layer.packed_weight.clone()
    with pytest.raises(RuntimeError, match="invalid INT4 state"):
        layer.load_state_dict(state)
    assert torch.equal(before, layer.packed_weight)       # nothing was copied


def test_checkpoint_roundtrip_dtype_pinning_and_no_alias():
    torch.manual_seed(14)
    w = torch.randn(7, 65, requires_grad=True)
    bias = torch.randn(7, requires_grad=True)
    layer = ops.QuantizedLinear.from_float(w, bias)
    assert not list(layer.parameters())
    assert not layer.scales.requires_grad and not layer.bias.requires_grad
    assert layer.bias.data_ptr() != bias.data_ptr()
    assert sorted(layer.state_dict()) == ["_extra_state", "bias", "packed_weight", "scales", "zeros"]
    scales = layer.scales.clone()
    for dtype in (torch.float16, torch.bfloat16, torch.float32):
        layer.to(dtype=dtype)
        assert layer.scales.dtype == torch.float32 and torch.equal(layer.scales, scales)
        assert layer.packed_weight.dtype == layer.zeros.dtype == torch.int32
    buffer = io.BytesIO()
    torch.save(layer.state_dict(), buffer)
    buffer.seek(0)
    clone = ops.QuantizedLinear.from_state_dict(torch.load(buffer, weights_only=True))
    for name in ("packed_weight", "scales", "zeros", "bias"):
        assert torch.equal(getattr(clone, name), getattr(layer, name))
    other = torch.nn.Sequential(ops.QuantizedLinear.from_float(torch.randn(7, 65), torch.zeros(7)))
    other.load_state_dict(torch.nn.Sequential(layer).state_dict())
    assert torch.equal(other[0].packed_weight, layer.packed_weight)


@pytest.mark.parametrize("field,value", [("format_version", 1), ("packing", "high_first"), ("group_size", 128),
                                         ("original_shape", [7, 66]), ("fp16_weight_rounding", "fp32")])
def test_reject_incompatible_metadata(field, value):
    layer = ops.QuantizedLinear.from_float(torch.randn(7, 65))
    state = copy.deepcopy(layer.state_dict())
    state["_extra_state"][field] = value
    with pytest.raises((ValueError, RuntimeError)):
        layer.load_state_dict(state)
    if field != "original_shape":
        with pytest.raises((ValueError, RuntimeError)):
            ops.QuantizedLinear.from_state_dict(state)


def test_no_cpu_compute_path():
    """Where the reference falls back to its CPU route, this package refuses."""
    layer = ops.QuantizedLinear.from_float(torch.ones(3, 65))
    x = torch.ones(1, 65, dtype=torch.float16)
    report = layer.execution_info(x)
    assert report["implementation"] == "unavailable" and "CUDA FP16" in report["fallback_reason"]
    assert report["input_copies"] == [] and report["format_version"] == 2
    for backend in ("auto", "cuda", "gemv", "small", "tensorcore", "naive", "reference"):
        layer.backend = backend
        with pytest.raises(ValueError, match="CUDA FP16"):
            layer(x)
    layer.backend = "bogus"
    with pytest.raises(ValueError, match="backend must be one of"):
        layer(x)
    with pytest.raises(ValueError, match="CUDA"):
        layer.dequantize()
    with pytest.raises(ValueError, match="CUDA"):
        ops.dequantize_int4(layer.packed_weight, layer.scales, layer.zeros, 65)
    with pytest.raises(ValueError, match="invalid quantized backend"):
        ops.QuantizedLinear(layer.packed_weight, layer.scales, layer.zeros, in_features=65, backend="bogus")
    with pytest.raises(ValueError, match="bits=4"):
        ops.QuantizedLinear.from_float(torch.ones(3, 8), bits=8)


def test_invalid_functional_metadata():
    layer = ops.QuantizedLinear.from_float(torch.randn(3, 65))
    x = torch.ones(2, 65, dtype=torch.float16)
    with pytest.raises(TypeError, match="scales"):
        ops.quantized_linear(x, layer.packed_weight, layer.scales.half(), layer.zeros, in_features=65)
    with pytest.raises(ValueError, match="shape"):
        ops.quantized_linear(x, layer.packed_weight, layer.scales[:, :1], layer.zeros, in_features=65)
    with pytest.raises(ValueError, match="bias"):
        ops.quantized_linear(x, layer.packed_weight, layer.scales, layer.zeros, in_features=65, bias=torch.ones(4))
    with pytest.raises(ValueError, match="in_features"):
        ops.quantized_linear(x[:, :64], layer.packed_weight, layer.scales, layer.zeros, in_features=65)
    with pytest.raises(TypeError, match="float16, bfloat16, or float32"):
        ops.quantized_linear(x.to(torch.int32), layer.packed_weight, layer.scales, layer.zeros, in_features=65)
    with pytest.raises(ValueError, match="in_features must be"):
        validate_int4_state(layer.packed_weight, layer.scales, layer.zeros, 0)


def test_ops_namespace_checks_run_before_any_device_work():
    layer = ops.QuantizedLinear.from_float(torch.randn(5, 65))
    x = torch.ones(1, 65, dtype=torch.float16)
    assert torch.ops.dandan_ops.w4a16_contract_version() == 2
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.dandan_ops.w4a16_gemv(x, layer.packed_weight, layer.scales, layer.zeros, 64)


def test_gemm_cost_model_picks_pair_kernels():
    """Shapes on which the measured cost model prefers each family."""
    assert _native.plan(512, 12288, 4096)["grid"] == 2 * 48 * 3         # pair, 192 rows of x per pair
    assert _native.plan(2048, 4096, 4096)["grid"] == 2 * 16 * 8         # pair, 256 rows of x per pair
    assert _native.plan(256, 24576, 4096)["grid"] == 128                # single CTA, 256 x 192
    small = _native.plan(100, 4096, 4096)                               # 16 tiles of one row: K split four ways
    assert small["route"] == "b200_tcgen05" and small["k_splits"] == 4 and small["grid"] == 2 * 16 * 4
    assert _native.plan(48, 57344, 8192)["route"] == "b200_tcgen05"     # large layer: the GEMM from 33 rows on
    assert _native.plan(32, 57344, 8192)["route"] == "b200_stream"
    assert _native.plan(48, 6144, 1024)["route"] == "b200_stream"       # small layer: streaming kernel up to 64 rows
    split = _native.plan(256, 4096, 28672)                              # 16 tiles, 112 blocks of K: four CTAs per tile
    assert split["k_splits"] == 4 and split["grid"] == 2 * 16 * 4


def test_operator_library_registers_the_reference_op_names():
    """The C++ operator library (TORCH_LIBRARY over the C ABI) builds without a GPU, loads with
    torch.ops.load_library and defines the reference's native op surface
    (dandan_ops/csrc/operators.cu:259-278, dandan_ops/csrc/hgemm.cu:89-98)."""
    import torch

    from dandan_ops_b200 import build as b2build
    from dandan_ops_b200 import ops as b2ops

    path = b2build.build_shim()
    assert path.is_file()
    import dandan_ops_b200  # noqa: F401  (registers on import)
    for name in ("w4a16_gemv", "w4a16_small", "w4a16_tensorcore", "w4a16_gemm", "w4a16_contract_version"):
        assert hasattr(torch.ops.dandan_ops, name)
    assert torch.ops.dandan_ops.w4a16_contract_version() == 2
    if b2ops.SHIM_LOADED:
        assert hasattr(torch.ops.dandan_ops, "w4a16_linear_image")
        schema = str(torch.ops.dandan_ops.w4a16_small.default._schema)
        assert "Tensor x, Tensor packed_w, Tensor scales, Tensor zeros, int group_size" in schema


def test_stream_plan_keeps_tickets_inside_the_ticket_area():
    """Host-only planning arithmetic: one arrival ticket per row tile of a split row group must fit in the
    workspace's ticket area (its last word is the status word), whatever the layer's height, and the workspace
    size grows with the partial tiles the plan needs."""
    from dandan_ops_b200 import _native

    lib = _native.load()
    tickets = _native.TICKET_BYTES // 4 - 1
    for n, k, m in ((200_000, 4096, 1), (1_000_000, 1024, 8), (131072, 8192, 16), (57344, 8192, 8), (8192, 28672, 1), (64, 64, 1)):
        plan = _native.plan(m, n, k)
        need = lib.b2_w4a16_workspace_bytes(m, n, k)
        assert need >= _native.TICKET_BYTES
        if plan["route"] == "b200_stream":
            groups16 = -(-(-(-n // 16)) // 16)
            if groups16 > plan["grid"]:                      # split row groups are indexed by CTA: grid * 16 tickets
                assert plan["grid"] * 16 <= tickets, (n, k, m, plan)
            assert plan["k_splits"] >= 1 and plan["grid"] >= 1


def test_gather_form_query_is_a_pure_function_of_the_problem():
    """`b2_w4a16_linear_gather_launches`: which calls run projection and gather as one kernel.  Needs no GPU
    (an unknown device counts as 148 SMs); every rank must get the same answer for equal slices."""
    q = _native.linear_gather_launches
    mailbox = 1 << 20
    # decode sizes of the 70B MLP on 8 ranks: the streaming kernel carries the exchange
    assert {q(m, 57344, 7168, 8192, r, 8, mailbox) for m in (1, 8, 16) for r in range(8)} == {1}
    assert {q(m, 8192, 1024, 28672, r, 8, mailbox) for m in (1, 8) for r in range(8)} == {1}
    # tile-kernel layers: one launch only while the last CTA collects in a single round of packets
    assert q(1, 4096, 2048, 1024, 0, 2, mailbox) == 1 and q(8, 4096, 2048, 1024, 0, 2, mailbox) == 2
    # more than 16 rows, or a slice that does not fit the mailbox: projection, then the gather kernel
    assert q(17, 57344, 7168, 8192, 0, 8, mailbox) == 2 and q(8, 57344, 7168, 8192, 0, 8, 1024) == 2
    # a rank without rows launches the gather alone; bad arguments give 0
    assert q(4, 100, 16, 64, 7, 8, mailbox) == 1
    assert q(0, 57344, 7168, 8192, 0, 8, mailbox) == 0 and q(8, 57344, 7168, 8192, 8, 8, mailbox) == 0
