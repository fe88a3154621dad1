"""The CPU oracle against the reference's own outputs on the benchmark configurations.

`golden/w4a16_configs.*` were written by `golden/make_config_golden.py`, which runs the reference's
Python package on its CPU route.  The oracle must reproduce the reference's state bit for bit and
its sampled outputs within the reference's acceptance rule |y - y_ref| <= 2e-3 + 2e-3*|y_ref|.
Only the configurations that numpy finishes in seconds are replayed here; the large ones are
replayed on the GPU by test_configs_gpu.py.
"""
import numpy as np
import pytest
import torch

import cases
from oracle import w4a16_oracle as oracle

ARR, META = cases.config_golden()


def _small(cfg):
    return [(cfg, si) for si, (_, n, k) in enumerate(cases.CONFIGS[cfg]["shapes"]) if n * k <= 32e6]


def test_fixture_inventory():
    assert {c: len(v) for c, v in META["configs"].items()} == {"cfg2": 4, "cfg3": 4, "cfg4": 2}
    assert len(META["stress"]) == 36 and len(META["n2"]) == 5
    for cfg, entries in META["configs"].items():
        for si, e in enumerate(entries):
            assert (e["name"], e["n"], e["k"]) == tuple(cases.CONFIGS[cfg]["shapes"][si])
            assert sorted(int(m) for m in e["ms"]) == cases.CONFIGS[cfg]["ms"]
            assert e["cols"] == cases.sample_columns(e["n"])


@pytest.mark.parametrize("cfg,si", _small("cfg2") + _small("cfg3"))
def test_oracle_reproduces_reference_on_quantized_configs(cfg, si):
    e = META["configs"][cfg][si]
    w, xs = cases.config_inputs(cfg, si)
    assert cases.sha(w) == e["sha_w"]
    codes, step, zero = oracle.quantize(w.numpy())
    words = oracle.pack(codes)
    assert cases.sha(words) == e["sha_words"] and cases.sha(step) == e["sha_step"] and cases.sha(zero) == e["sha_zero"]
    assert cases.sha(oracle.dequantize_fp16(words, step, zero, e["k"])) == e["sha_deq_fp16"]
    cols = np.array(e["cols"])
    for m, x in xs.items():
        assert cases.sha(x) == e["ms"][str(m)]["sha_x"]
        rows = np.array(e["ms"][str(m)]["rows"])
        y = oracle.linear(x.numpy()[rows], words[cols], step[cols], zero[cols], e["k"])
        assert oracle.within_tolerance(y, ARR[f"{cfg}_{si}_m{m}_y"])


@pytest.mark.parametrize("case", [c for c in META["stress"] if c["n"] * c["k"] <= 40e6], ids=lambda c: f"cfg5_{c['idx']}")
def test_oracle_reproduces_reference_on_the_stress_sweep(case):
    n, k, m, seed = case["n"], case["k"], case["m"], case["seed"]
    words, step, zero = cases.direct_state(n, k, seed, lambda c: torch.from_numpy(oracle.pack(c.numpy())))
    x = cases.stress_x(m, k, seed)
    assert cases.sha(words) == case["sha_words"] and cases.sha(step) == case["sha_step"]
    assert cases.sha(zero) == case["sha_zero"] and cases.sha(x) == case["sha_x"]
    words, step, zero = words.numpy(), step.numpy(), zero.numpy()
    if n * k <= 13e6:
        assert cases.sha(oracle.dequantize_fp16(words, step, zero, k)) == case["sha_deq_fp16"]
    cols = np.array(case["cols"])
    y = oracle.linear(x.numpy(), words[cols], step[cols], zero[cols], k)
    assert oracle.within_tolerance(y, ARR[f"cfg5_{case['idx']}_y"])


@pytest.mark.parametrize("case", META["n2"], ids=lambda c: f"n2_{c['idx']}")
def test_oracle_reproduces_reference_formulas_around_the_projection(case):
    """residual + RMSNorm and SiLU*mul: the FP16 sum is exact; the normalized values and the
    activation may land on the neighbouring FP16 number where the FP32 mean or exp differ in the
    last bit (tolerance: 2e-3 relative = two FP16 ulps, on at most 0.5 % of the elements)."""
    i, m, k = case["idx"], case["m"], case["k"]
    x, res, wn, gate, up = cases.n2_inputs(i, m, k)
    for eps in case["eps"]:
        tag = f"n2_norm_{i}_{eps:g}"
        out, summed = oracle.residual_rms_norm(x.numpy(), res.numpy(), wn.numpy(), eps)
        assert np.array_equal(summed.view(np.uint16), ARR[tag + "_sum"].view(np.uint16))
        np.testing.assert_allclose(out.astype(np.float64), ARR[tag + "_out"].astype(np.float64), rtol=2e-3, atol=1e-6)
        assert np.mean(out != ARR[tag + "_out"]) < 5e-3
    got = oracle.silu_and_mul(gate.numpy(), up.numpy())
    np.testing.assert_allclose(got.astype(np.float64), ARR[f"n2_silu_{i}"].astype(np.float64), rtol=2e-3, atol=1e-7)
    assert np.mean(got != ARR[f"n2_silu_{i}"]) < 5e-3
