"""Generate the committed golden fixtures by running the reference's own Python code.

Usage (only where the reference checkout is available):

    python tests/golden/make_golden.py /path/to/reference

It imports `dandan_ops` from that checkout (its CPU route needs no compiled
extension), runs the quantizer, packer, dequantizer and the CPU forward on seeded
inputs and stores the results next to this script:

  w4a16_golden.npz   full tensors for the small cases
  w4a16_golden.json  case descriptions and SHA-256 digests for the large ones

The tests never import the reference; they read these two files.
"""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def digest(t):
    a = t.detach().cpu().contiguous().numpy() if isinstance(t, torch.Tensor) else np.ascontiguousarray(t)
    return hashlib.sha256(a.tobytes()).hexdigest()


def edge_weight(kind, k):
    torch.manual_seed(k)
    w = torch.randn(3, k)
    if kind == "zero":
        w.zero_()
    elif kind == "constant":
        w.fill_(2.5)
    elif kind == "positive":
        w.abs_()
    elif kind == "negative":
        w = -w.abs()
    elif kind == "tiny":
        w *= 1e-39
    elif kind == "large":
        w *= 1e30
    return w


def direct_state(ops, n, k, seed):
    """State built without the quantizer: uniform codes and zero points, log-normal
    FP16-representable steps with 1 % of the groups enlarged fifty-fold."""
    g = torch.Generator().manual_seed(seed)
    groups = (k + 63) // 64
    codes = torch.randint(0, 16, (n, k), generator=g, dtype=torch.uint8)
    zero = torch.randint(0, 16, (n, groups), generator=g, dtype=torch.int32)
    step = torch.exp(torch.randn(n, groups, generator=g) * 0.5 - 5.0)
    outlier = torch.rand(n, groups, generator=g) < 0.01
    step = torch.where(outlier, step * 50.0, step).half().float()
    return ops.pack_int4(codes), step, zero


def main(ref_root):
    sys.path.insert(0, ref_root)
    import dandan_ops as ops

    arrays, meta = {}, {"cases": {}}

    # 1. nibble order known-answer (reference tests/test_quantized_contract.py:38-42)
    q = torch.tensor([[0, 1, 2, 3, 4, 5, 6, 15, 9]], dtype=torch.uint8)
    arrays["kat_codes"] = q.numpy()
    arrays["kat_words"] = ops.pack_int4(q).numpy()

    # 2. quantizer edge cases (reference tests/test_quantized_contract.py:12-35)
    edges = []
    for k in (1, 7, 8, 9, 63, 64, 65, 127, 128, 129):
        for kind in ("zero", "constant", "positive", "negative", "tiny", "large"):
            w = edge_weight(kind, k)
            codes, step, zero = ops.quantize_int4(w)
            words = ops.pack_int4(codes)
            tag = f"edge_{kind}_{k}"
            arrays[tag + "_w"] = w.numpy()
            arrays[tag + "_codes"] = codes.numpy()
            arrays[tag + "_step"] = step.numpy()
            arrays[tag + "_zero"] = zero.numpy()
            arrays[tag + "_words"] = words.numpy()
            arrays[tag + "_deq"] = ops.dequantize_int4(words, step, zero, k).numpy()
            edges.append([kind, k])
    meta["edges"] = edges

    # 3. small linear cases with full tensors
    small = []
    for name, n, k, m, seed, with_bias, dtype in (
            ("lin_67x129", 67, 129, 3, 51, False, torch.float16),
            ("lin_7x65_bias", 7, 65, 4, 7, True, torch.float32),
            ("lin_37x257", 37, 257, 8, 302, False, torch.float16),
            ("lin_5x1", 5, 1, 1, 6, False, torch.float16),
            ("lin_33x64", 33, 64, 17, 114, False, torch.float16)):
        torch.manual_seed(seed)
        w = torch.randn(n, k, dtype=dtype)
        bias = torch.randn(n) if with_bias else None
        layer = ops.QuantizedLinear.from_float(w, bias)
        x = torch.randn(m, k, dtype=torch.float16)
        arrays[name + "_w"] = w.numpy()
        arrays[name + "_x"] = x.numpy()
        arrays[name + "_words"] = layer.packed_weight.numpy()
        arrays[name + "_step"] = layer.scales.numpy()
        arrays[name + "_zero"] = layer.zeros.numpy()
        arrays[name + "_y"] = layer(x).numpy()
        if bias is not None:
            arrays[name + "_bias"] = bias.numpy()
        small.append({"name": name, "n": n, "k": k, "m": m, "bias": with_bias})
    meta["small"] = small

    # 4. the CPU-runnable benchmark configuration: W [2048,1024] ~ N(0, 0.02^2), x [8,1024]
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(2048, 1024, generator=g) * 0.02).half()
    x = torch.randn(8, 1024, generator=g).half()
    layer = ops.QuantizedLinear.from_float(w, group_size=64)
    y = layer(x)
    arrays["cfg1_x"] = x.numpy()
    arrays["cfg1_y"] = y.numpy()
    meta["cases"]["cfg1"] = {
        "n": 2048, "k": 1024, "m": 8, "seed": 0, "sigma": 0.02,
        "sha_w": digest(w), "sha_words": digest(layer.packed_weight),
        "sha_step": digest(layer.scales), "sha_zero": digest(layer.zeros),
        "sha_deq_fp16": digest(layer.dequantize().half()),
        "storage_bytes": int(layer.storage_bytes),
        "info": layer.execution_info(x),
    }

    # 5. direct-state stress cases (tails in N, several M)
    stress = []
    for idx, (n, k, m) in enumerate(((1000, 1024, 3), (12289, 1024, 1), (1000, 3072, 17), (4096, 1024, 100))):
        seed = 4000 + idx
        words, step, zero = direct_state(ops, n, k, seed)
        g = torch.Generator().manual_seed(seed + 500)
        x = torch.randn(m, k, generator=g).half()
        layer = ops.QuantizedLinear(words, step, zero, in_features=k)
        y = layer(x)
        name = f"stress{idx}"
        col_step = 16 if m * n > 100000 else 1      # keep the fixture small: every 16th column
        arrays[name + "_y"] = np.ascontiguousarray(y.numpy()[:, ::col_step])
        stress.append({"name": name, "n": n, "k": k, "m": m, "seed": seed, "col_step": col_step,
                       "sha_words": digest(words), "sha_step": digest(step),
                       "sha_zero": digest(zero), "sha_x": digest(x),
                       "sha_deq_fp16": digest(layer.dequantize().half())})
    meta["stress"] = stress

    # 6. module metadata the drop-in must reproduce
    layer = ops.QuantizedLinear.from_float(torch.ones(3, 65))
    meta["extra_state"] = layer.get_extra_state()
    meta["backends"] = list(__import__("dandan_ops.quantized_linear", fromlist=["BACKENDS"]).BACKENDS)
    meta["torch"] = torch.__version__

    np.savez_compressed(HERE / "w4a16_golden.npz", **arrays)
    (HERE / "w4a16_golden.json").write_text(json.dumps(meta, indent=1, sort_keys=True) + "\n")
    print("wrote", len(arrays), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
