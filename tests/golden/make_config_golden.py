"""Generate the fixtures of the benchmark configurations by running the reference's own code.

Usage (only where the reference checkout is available; needs ~12 GB of host memory and a few
minutes on eight cores):

    python tests/golden/make_config_golden.py /path/to/reference

For every projection of the Qwen3-0.6B, Qwen3-8B and Llama-3-70B configurations (seeds
1000/2000/3000 + shape index) the reference quantizes the seeded weight on its CPU route and the
script stores SHA-256 digests of `packed_weight`, `scales`, `zeros` and `dequantize().half()`,
plus the reference's CPU forward output on a fixed sample of output columns (and of the rows of x
for large batches): the sampled columns are run through the reference as a layer built from the
corresponding rows of its own state.  For the 36 cases of the stress sweep (seed 4000 + case
index, state built directly, not quantized) it stores the same digests and sampled outputs.  The
formulas either side of the projection (`residual_rms_norm`, `silu_and_mul`, CPU route) are
pinned on seeded inputs as well.

Writes w4a16_configs.npz (sampled outputs) and w4a16_configs.json (digests, sample indices).
The tests never import the reference; they read these two files.
"""
import json
import sys
import time
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import cases  # noqa: E402


def main(ref_root):
    sys.path.insert(0, ref_root)
    import dandan_ops as ops
    from dandan_ops import elementwise

    torch.set_num_threads(8)
    arrays, meta = {}, {"configs": {}, "stress": [], "n2": []}

    for cfg, spec in cases.CONFIGS.items():
        entries = []
        for si, (name, n, k) in enumerate(spec["shapes"]):
            t0 = time.time()
            w, xs = cases.config_inputs(cfg, si)
            layer = ops.QuantizedLinear.from_float(w, group_size=64)
            cols = cases.sample_columns(n)
            idx = torch.tensor(cols)
            sub = ops.QuantizedLinear(layer.packed_weight[idx], layer.scales[idx], layer.zeros[idx], in_features=k)
            entry = {"name": name, "n": n, "k": k, "seed": spec["seed"] + si, "sigma": spec["sigma"],
                     "sha_w": cases.sha(w), "sha_words": cases.sha(layer.packed_weight),
                     "sha_step": cases.sha(layer.scales), "sha_zero": cases.sha(layer.zeros),
                     "sha_deq_fp16": cases.sha(layer.dequantize().half()), "cols": cols, "ms": {}}
            for m, x in xs.items():
                rows = cases.sample_rows(m)
                y = sub(x[torch.tensor(rows)])
                assert sub.execution_info(x)["implementation"] == "reference"
                arrays[f"{cfg}_{si}_m{m}_y"] = y.numpy()
                entry["ms"][str(m)] = {"rows": rows, "sha_x": cases.sha(x)}
            entries.append(entry)
            print(cfg, name, n, k, f"{time.time() - t0:.1f}s", flush=True)
            del w, xs, layer, sub
        meta["configs"][cfg] = entries

    for idx, n, k, m in cases.stress_cases():
        seed = 4000 + idx
        words, step, zero = cases.direct_state(n, k, seed, ops.pack_int4)
        x = cases.stress_x(m, k, seed)
        cols = cases.sample_columns(n)
        ci = torch.tensor(cols)
        sub = ops.QuantizedLinear(words[ci], step[ci], zero[ci], in_features=k)
        arrays[f"cfg5_{idx}_y"] = sub(x).numpy()
        full = ops.QuantizedLinear(words, step, zero, in_features=k)
        meta["stress"].append({"idx": idx, "n": n, "k": k, "m": m, "seed": seed, "cols": cols,
                               "sha_words": cases.sha(words), "sha_step": cases.sha(step), "sha_zero": cases.sha(zero),
                               "sha_x": cases.sha(x), "sha_deq_fp16": cases.sha(full.dequantize().half())})
        print("cfg5", idx, n, k, m, flush=True)

    # the formulas either side of the projection, reference CPU route
    for i, (m, k) in enumerate(((1, 1024), (8, 4096), (16, 1024), (5, 8192), (64, 2048))):
        x, res, wn, gate, up = cases.n2_inputs(i, m, k)
        for eps in (1e-5, 1e-6):
            normed, summed = elementwise.residual_rms_norm(x, res, wn, eps)
            tag = f"n2_norm_{i}_{eps:g}"
            arrays[tag + "_out"], arrays[tag + "_sum"] = normed.numpy(), summed.numpy()
        arrays[f"n2_silu_{i}"] = elementwise.silu_and_mul(gate, up).numpy()
        meta["n2"].append({"idx": i, "m": m, "k": k, "seed": 5000 + i, "eps": [1e-5, 1e-6]})

    meta["torch"] = torch.__version__
    np.savez_compressed(HERE / "w4a16_configs.npz", **arrays)
    (HERE / "w4a16_configs.json").write_text(json.dumps(meta, sort_keys=True) + "\n")
    print("wrote", len(arrays), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
