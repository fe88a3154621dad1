"""The CUDA engine on every benchmark configuration at its own shapes, seeds and batch sizes,
against outputs of the reference itself (`golden/w4a16_configs.*`, written by
`golden/make_config_golden.py` from the reference's CPU route).

Per projection: the quantized state and the dequantized FP16 weights must equal the reference's
bit for bit (SHA-256); per batch size the output must satisfy the reference's acceptance rule
|y - y_ref| <= 2e-3 + 2e-3*|y_ref| on the sampled columns the fixture holds, and on EVERY
column against an FP32 product of the (bit-verified) FP16 weights computed with torch on the GPU.
Every call goes through the C ABI with the output and the workspace embedded in buffers whose
margins hold a sentinel, so a store outside either is seen; tickets must be zero again and the
status word clear after each call.  max_abs / relative_l2 / mismatch fraction per case are
appended to the JSON file named by B2_PARITY_REPORT when that variable is set.
"""
import json
import os

import numpy as np
import pytest
import torch

import cases
import dandan_ops_b200 as ops
from dandan_ops_b200 import _native

pytestmark = pytest.mark.gpu
ARR, META = cases.config_golden()
MARGIN = 4096            # sentinel elements (y) / bytes (workspace) either side
SENTINEL16 = 0x7B5A      # an FP16 bit pattern no output of these cases takes (~60 000)


def _report(name, m, metrics, extra=None):
    path = os.environ.get("B2_PARITY_REPORT")
    if not path:
        return
    row = {"case": name, "M": m, **metrics, **(extra or {})}
    with open(path, "a") as f:
        f.write(json.dumps(row) + "\n")


def guarded_linear(x, image, n, k, route=_native.ROUTE_AUTO):
    """b2_w4a16_linear_route straight through the C ABI with sentinel margins around y and around a
    workspace of exactly b2_w4a16_workspace_bytes; returns y after checking margins, tickets, status."""
    lib = _native.load()
    m = x.shape[0]
    ybuf = torch.full((m * n + 2 * MARGIN,), SENTINEL16, dtype=torch.int16, device="cuda")
    y = ybuf[MARGIN:MARGIN + m * n].view(torch.float16).view(m, n)
    need = int(lib.b2_w4a16_workspace_bytes(m, n, k))
    assert need >= _native.TICKET_BYTES
    wbuf = torch.full((need + 2 * MARGIN,), 0xA5, dtype=torch.uint8, device="cuda")
    ws = wbuf[MARGIN:MARGIN + need]
    ws[:_native.TICKET_BYTES].zero_()
    assert ws.data_ptr() % 16 == 0
    rc = lib.b2_w4a16_linear_route(x.data_ptr(), x.stride(0) if m > 1 else k, image.data_ptr(), y.data_ptr(), n,
                                   m, n, k, ws.data_ptr(), need, torch.cuda.current_stream().cuda_stream, route)
    assert rc == 0, lib.b2_w4a16_last_error()
    torch.cuda.synchronize()
    assert bool((ybuf[:MARGIN] == SENTINEL16).all()) and bool((ybuf[MARGIN + m * n:] == SENTINEL16).all()), "store outside y"
    assert bool((wbuf[:MARGIN] == 0xA5).all()) and bool((wbuf[MARGIN + need:] == 0xA5).all()), "store outside the workspace"
    assert not bool(ws[:_native.TICKET_BYTES].any()), "tickets or status word left non-zero"
    assert not bool((ybuf[MARGIN:MARGIN + m * n] == SENTINEL16).any()), "an output element was never written"
    return y


def check_outputs(name, y, x, w16, cols, rows, y_ref, m):
    """Sampled columns against the reference's output, every column against the FP32 product."""
    got = y[torch.tensor(rows, device="cuda")][:, torch.tensor(cols, device="cuda")].cpu().numpy()
    metrics = cases.error_metrics(got, y_ref)
    full_ref = (x.float() @ w16.float().t())
    diff = (y.float() - full_ref).abs()
    full_ratio = float((diff / (2e-3 + 2e-3 * full_ref.abs())).max())
    _report(name, m, metrics, {"all_columns_bound_ratio": full_ratio, "all_columns_max_abs": float(diff.max())})
    assert metrics["bound_ratio"] <= 1.0, metrics
    assert full_ratio <= 1.0, full_ratio


@pytest.mark.parametrize("cfg,si", [(c, i) for c in ("cfg2", "cfg3", "cfg4") for i in range(len(cases.CONFIGS[c]["shapes"]))])
def test_quantized_configuration_at_its_own_shapes(cfg, si):
    e = META["configs"][cfg][si]
    n, k = e["n"], e["k"]
    w, xs = cases.config_inputs(cfg, si)
    assert cases.sha(w) == e["sha_w"]
    layer = ops.QuantizedLinear.from_float(w.cuda(), group_size=64)
    del w
    assert cases.sha(layer.packed_weight) == e["sha_words"]
    assert cases.sha(layer.scales) == e["sha_step"] and cases.sha(layer.zeros) == e["sha_zero"]
    w16 = layer.dequantize().half()
    assert cases.sha(w16) == e["sha_deq_fp16"]
    image = layer._native_image()
    for m, x in xs.items():
        assert cases.sha(x) == e["ms"][str(m)]["sha_x"]
        xg = x.cuda()
        y = guarded_linear(xg, image, n, k)
        assert torch.equal(y, layer(xg))                       # the module's forward is the same call
        check_outputs(f"{cfg}/{e['name']}_{n}x{k}", y, xg, w16, e["cols"], e["ms"][str(m)]["rows"],
                      ARR[f"{cfg}_{si}_m{m}_y"], m)
        if m <= 16 and cfg != "cfg2":                           # the streaming kernel's split-K at full size as well
            y2 = guarded_linear(xg, image, n, k, route=_native.ROUTE_STREAM)
            check_outputs(f"{cfg}/{e['name']}_{n}x{k}/stream", y2, xg, w16, e["cols"], e["ms"][str(m)]["rows"],
                          ARR[f"{cfg}_{si}_m{m}_y"], m)


@pytest.mark.parametrize("case", META["stress"], ids=lambda c: f"cfg5_{c['idx']}_{c['n']}x{c['k']}_m{c['m']}")
def test_stress_sweep_every_case(case):
    n, k, m, seed = case["n"], case["k"], case["m"], case["seed"]
    words, step, zero = cases.direct_state(n, k, seed, lambda c: ops.pack_int4(c.cuda()).cpu())
    assert cases.sha(words) == case["sha_words"] and cases.sha(step) == case["sha_step"] and cases.sha(zero) == case["sha_zero"]
    layer = ops.QuantizedLinear(words.cuda(), step.cuda(), zero.cuda(), in_features=k)
    w16 = layer.dequantize().half()
    assert cases.sha(w16) == case["sha_deq_fp16"]
    x = cases.stress_x(m, k, seed)
    assert cases.sha(x) == case["sha_x"]
    xg = x.cuda()
    y = guarded_linear(xg, layer._native_image(), n, k)
    assert torch.equal(y, layer(xg))
    check_outputs(f"cfg5/{case['idx']}_{n}x{k}", y, xg, w16, case["cols"], list(range(m)), ARR[f"cfg5_{case['idx']}_y"], m)
    if m <= 16:
        y2 = guarded_linear(xg, layer._native_image(), n, k, route=_native.ROUTE_STREAM)
        check_outputs(f"cfg5/{case['idx']}_{n}x{k}/stream", y2, xg, w16, case["cols"], list(range(m)),
                      ARR[f"cfg5_{case['idx']}_y"], m)


@pytest.mark.parametrize("case", META["n2"], ids=lambda c: f"n2_{c['idx']}")
def test_formulas_around_the_projection_against_the_reference(case):
    """Residual + RMSNorm kernel and the SiLU*mul pair kernel against the reference's CPU outputs.
    The FP16 sum is exact.  The FP32 sum of squares is added in another order and expf differs from
    the CPU's exp in the last bit now and then, so a value may land on the neighbouring FP16 number:
    tolerance 2e-3 relative (two FP16 ulps), on at most 0.5 % of the elements."""
    i, m, k = case["idx"], case["m"], case["k"]
    x, res, wn, gate, up = (t.cuda() for t in cases.n2_inputs(i, m, k))
    for eps in case["eps"]:
        tag = f"n2_norm_{i}_{eps:g}"
        out, summed = _native.residual_rms_norm(x, res, wn, eps)
        assert np.array_equal(summed.cpu().numpy().view(np.uint16), ARR[tag + "_sum"].view(np.uint16))
        got = out.cpu().numpy()
        np.testing.assert_allclose(got.astype(np.float64), ARR[tag + "_out"].astype(np.float64), rtol=2e-3, atol=1e-6)
        assert np.mean(got != ARR[tag + "_out"]) < 5e-3
    # gate/up in pair order: columns 16j..16j+7 gate, 16j+8..16j+15 up of outputs 8j..8j+7
    pairs = torch.stack((gate.view(m, k // 8, 8), up.view(m, k // 8, 8)), dim=2).reshape(m, 2 * k).contiguous()
    got = _native.silu_mul_pairs(pairs).cpu().numpy()
    np.testing.assert_allclose(got.astype(np.float64), ARR[f"n2_silu_{i}"].astype(np.float64), rtol=2e-3, atol=1e-7)
    assert np.mean(got != ARR[f"n2_silu_{i}"]) < 5e-3
