"""Pins the numpy oracle to fixtures produced by the reference's own Python code."""
import numpy as np
import pytest
import torch

import cases
from oracle import w4a16_oracle as oracle

ARR, META = cases.golden()


def test_nibble_order_known_answer():
    codes = np.array([[0, 1, 2, 3, 4, 5, 6, 15, 9]], dtype=np.uint8)
    words = oracle.pack(codes)
    assert words.tolist() == [[0xF6543210 - 2**32, 9]]
    assert np.array_equal(words, ARR["kat_words"])
    assert np.array_equal(oracle.unpack(words, 9), codes)


@pytest.mark.parametrize("kind,k", [tuple(e) for e in META["edges"]])
def test_quantizer_edges_bit_exact(kind, k):
    tag = f"edge_{kind}_{k}"
    w = ARR[tag + "_w"]
    assert np.array_equal(w, cases.edge_weight(kind, k).numpy())
    codes, step, zero = oracle.quantize(w)
    assert np.array_equal(codes, ARR[tag + "_codes"])
    assert np.array_equal(step.view(np.uint32), ARR[tag + "_step"].view(np.uint32))
    assert np.array_equal(zero, ARR[tag + "_zero"])
    words = oracle.pack(codes)
    assert np.array_equal(words, ARR[tag + "_words"])
    assert np.array_equal(oracle.unpack(words, k), codes)
    deq = oracle.dequantize(words, step, zero, k)
    assert np.array_equal(deq.view(np.uint32), ARR[tag + "_deq"].view(np.uint32))
    group = np.arange(k) // 64
    if kind == "zero":
        assert not deq.any()
    elif kind != "tiny":
        bound = step[:, group].astype(np.float64) * 1.01 + 1e-6
        assert (np.abs(deq.astype(np.float64) - w.astype(np.float64)) <= bound).all()


@pytest.mark.parametrize("case", META["small"], ids=lambda c: c["name"])
def test_small_linear_cases(case):
    name, k = case["name"], case["k"]
    codes, step, zero = oracle.quantize(ARR[name + "_w"])
    words = oracle.pack(codes)
    assert np.array_equal(words, ARR[name + "_words"])
    assert np.array_equal(step.view(np.uint32), ARR[name + "_step"].view(np.uint32))
    assert np.array_equal(zero, ARR[name + "_zero"])
    bias = ARR[name + "_bias"] if case["bias"] else None
    y = oracle.linear(ARR[name + "_x"], words, step, zero, k, bias=bias)
    assert oracle.within_tolerance(y, ARR[name + "_y"])
    # K this small sums in one BLAS panel: in practice the results are identical
    assert np.mean(y != ARR[name + "_y"]) < 0.02


def test_cpu_runnable_config_matches_reference():
    c = META["cases"]["cfg1"]
    w, x = cases.gaussian_case(c["n"], c["k"], c["m"], c["seed"], c["sigma"])
    assert cases.sha(w) == c["sha_w"]
    assert np.array_equal(x.numpy(), ARR["cfg1_x"])
    codes, step, zero = oracle.quantize(w.numpy())
    words = oracle.pack(codes)
    assert cases.sha(words) == c["sha_words"]
    assert cases.sha(step) == c["sha_step"]
    assert cases.sha(zero) == c["sha_zero"]
    assert cases.sha(oracle.dequantize_fp16(words, step, zero, c["k"])) == c["sha_deq_fp16"]
    assert oracle.storage_bytes(c["n"], c["k"]) == c["storage_bytes"]
    y = oracle.linear(x.numpy(), words, step, zero, c["k"])
    assert oracle.within_tolerance(y, ARR["cfg1_y"])
    y64 = oracle.linear_f64(x.numpy(), words, step, zero, c["k"])
    assert np.abs(ARR["cfg1_y"].astype(np.float64) - y64).max() < 2e-3


@pytest.mark.parametrize("case", META["stress"], ids=lambda c: c["name"])
def test_direct_state_stress(case):
    n, k, m = case["n"], case["k"], case["m"]
    pack = lambda codes: torch.from_numpy(oracle.pack(codes.numpy()))
    words, step, zero = cases.direct_state(n, k, case["seed"], pack)
    assert cases.sha(words) == case["sha_words"]
    assert cases.sha(step) == case["sha_step"]
    assert cases.sha(zero) == case["sha_zero"]
    x = cases.stress_x(m, k, case["seed"])
    assert cases.sha(x) == case["sha_x"]
    wn, sn, zn = words.numpy(), step.numpy(), zero.numpy()
    assert cases.sha(oracle.dequantize_fp16(wn, sn, zn, k)) == case["sha_deq_fp16"]
    y = oracle.linear(x.numpy(), wn, sn, zn, k)[:, ::case["col_step"]]
    assert oracle.within_tolerance(y, ARR[case["name"] + "_y"])


def test_torch_restatement_agrees_with_numpy():
    w, x = cases.gaussian_case(96, 200, 5, 77)
    codes, step, zero = oracle.quantize(w.numpy())
    words = oracle.pack(codes)
    y_np = oracle.linear(x.numpy(), words, step, zero, 200)
    y_t = oracle.torch_forward(x, torch.from_numpy(words), torch.from_numpy(step), torch.from_numpy(zero), 200)
    assert oracle.within_tolerance(y_t.numpy(), y_np)


def test_fp16_rounding_of_the_weights_is_part_of_the_contract():
    """The reference rounds every dequantized weight to FP16 before the product.  A kernel that applies
    the FP32 step to sums of integer differences instead (no per-weight rounding: closer to exact
    arithmetic, and 2.4 x fewer dequantization instructions) leaves the reference's own tolerance on
    the reference's own fixture - which is why the decode kernels keep the exact per-weight chain."""
    name, n, k = "lin_67x129", 67, 129
    words, step, zero = ARR[name + "_words"], ARR[name + "_step"], ARR[name + "_zero"]
    x, y_ref = ARR[name + "_x"], ARR[name + "_y"]
    group = np.arange(k) // 64
    diff = oracle.unpack(words, k).astype(np.float64) - zero[:, group].astype(np.float64)
    unrounded = diff * step[:, group].astype(np.float64)                     # no FP16 rounding of the weights
    y = (x.astype(np.float64) @ unrounded.T).astype(np.float16)
    assert not oracle.within_tolerance(y, y_ref)
    rounded = oracle.dequantize_fp16(words, step, zero, k).astype(np.float64)
    assert oracle.within_tolerance((x.astype(np.float64) @ rounded.T).astype(np.float16), y_ref)
