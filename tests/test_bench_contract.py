"""The benchmark's reference arm runs on host cores only, so its output contract is checked here;
the GPU arm's JSON line is produced by the same code path and checked for the shared keys when a
GPU is present."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
SHARED = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
          "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"}


def _last_json(stdout):
    lines = [l for l in stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, stdout
    return json.loads(lines[0])


def test_reference_arm_prints_one_contract_line():
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                          capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr
    line = _last_json(proc.stdout)
    assert SHARED <= set(line) and line["impl"] == "reference"
    assert line["metric"] == "w4a16_decode_weight_hbm_GBps" and line["unit"] == "GB/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["config"]["workload"] == "llama3-70b-mlp" and line["vs_baseline"] is None
    assert line["scaling"] == "strong"
    cpu = line["cpu_baseline"]
    # "reference" where a checkout of the reference can be imported, else the oracle's port of its CPU route
    assert cpu["kind"] in ("port", "reference") and cpu["cores"] >= 1 and cpu["value"] == line["value"] and cpu["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


@pytest.mark.gpu
def test_gpu_arm_prints_one_contract_line():
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--steps", "2", "--warmup", "3", "--no-cpu", "--workload-only"],
                          capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = _last_json(proc.stdout)
    assert SHARED | {"roofline", "gpu_launches", "clocks", "roofline_prefill", "floor_us", "parity"} <= set(line)
    assert line["config"]["workload"] == "llama3-70b-mlp" and line["scaling"] == "strong"
    roof = line["roofline"]
    assert roof["bound"] == "hbm" and 0 < roof["frac"] < 1.2 and roof["unit"] == "GB/s" and roof["traffic"] > 0
    assert roof["kernel"] == "w4a16_stream_kernel"
    assert line["gpu_launches"] == 2 * 24 and line["n_gpus"] == 1 and line["dtype"] == "f16"
    assert line["parity"]["ok"] is True and line["parity"]["linears_checked"] == 4 and line["status_word"] == 0
    assert 0 < line["floor_us"]["per_launch"] < 50
    e2e = line["e2e"]
    assert e2e["value"] > 0 and e2e["h2d_bytes_per_step"] > 0 and e2e["d2h_bytes_per_step"] > 0 and e2e["eager"]["value"] > 0
    pre = line["roofline_prefill"]
    assert pre["bound"] == "tensor" and pre["unit"] == "TFLOP/s" and 0 < pre["frac"] < 1.2


def test_clock_sampler_holds_the_load_until_samples_arrive():
    """The sampler keeps replaying the step until nvidia-smi has delivered its samples, and gives up
    after its time limit when it never does (no GPU needed: the sampler process is faked)."""
    sys.path.insert(0, str(ROOT))
    import bench

    sampler = bench.ClockSampler(0)
    assert sampler.summary()["samples"] == 0
    sampler.hold_load(lambda: pytest.fail("no sampler process: nothing to wait for"), lambda: None, 1, 1.0)

    sampler.proc = object()                      # "running"
    steps = []

    def run():
        steps.append(1)
        if len(steps) == 24:                     # the first sample arrives during the third batch of replays
            sampler.lines.append("1965, 1965, Not Active, Not Active, Not Active, Active\n")

    sampler.hold_load(run, lambda: None, 1, 30.0)
    assert len(steps) == 24 and sampler.summary() == {
        "sm_mhz": 1965.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 1,
        "window": sampler.summary()["window"]}

    import time
    t0 = time.monotonic()
    sampler.hold_load(lambda: None, lambda: time.sleep(0.01), 5, 0.2)    # never reaches five samples
    assert 0.2 <= time.monotonic() - t0 < 2.0
