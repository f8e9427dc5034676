"""The one-line JSON contract of bench.py: the CPU (reference) arm here, the CUDA arm on a GPU."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE_KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
             "vs_baseline", "dtype", "data", "config", "e2e"}


def _run(*flags):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *flags], capture_output=True, text=True,
                       timeout=900, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, r.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_line():
    d = _run("--impl", "reference", "--model", "tiny", "--cpu-batch", "2", "--steps", "1", "--warmup", "1")
    assert BASE_KEYS <= set(d) and d["impl"] == "reference"
    assert d["metric"] == "images/sec" and d["unit"] == "images/s" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["e2e"]["value"] == d["value"]
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    assert "workload" in d["config"] and "model" not in d["config"]


@pytest.mark.gpu
def test_cuda_arm_line():
    d = _run("--batch", "32", "--steps", "3", "--warmup", "3", "--cpu-batch", "2")
    assert BASE_KEYS <= set(d) and "impl" not in d
    assert d["metric"] == "images/sec" and d["dtype"] == "bf16" and d["n_gpus"] == 1 and d["scaling"] == "weak"
    assert d["value"] > 0 and d["vs_baseline"] is None and d["device_status"] == 0
    assert 0 < d["e2e"]["value"] <= d["value"] * 1.05
    # host images are fp32 by default (what the reference's loader hands over); bf16 is the secondary figure
    assert d["e2e"]["h2d_bytes_per_step"] == 32 * 3 * 256 * 256 * 4 and d["e2e"]["d2h_bytes_per_step"] == 32 * 1000 * 4
    assert d["config"]["e2e_host_images"] == "float32" and d["e2e_other_host_dtype"]["host_images"] == "bfloat16"
    assert d["gpu_launches"] == 3 * (9 + 7 * 12)      # DeiT-S: q and kv projections share a launch
    rf = d["roofline"]
    assert rf["bound"] == "tensor" and rf["unit"] == "TFLOP/s" and rf["peak"] > 0
    assert abs(rf["frac"] - rf["achieved"] / rf["peak"]) < 2e-3 and rf["traffic"] > 0
    assert 0 < rf["frac_all_launches"] < 1.5
    # the per-kernel estimates add up to the measured step
    blk = d["block"]
    assert abs(blk["depth"] * blk["block_ms_in_step_est"] + blk["front_back_ms"] - d["ms_per_step"]) < 0.02 * d["ms_per_step"]
    in_model = sum(k["ms_in_step_est"] for k in d["kernels"] if "note" not in k)
    assert abs(in_model - blk["block_ms_in_step_est"]) < 0.03 * blk["block_ms_in_step_est"] + 0.002   # rounded to 1e-4 ms
    assert 0 < d["model_roofline"]["frac"] < 1.5
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["value"] > 0 and cb["cores"] >= 1
    assert {"sm_mhz", "sm_max_mhz", "reasons"} <= set(d["clocks"])
    assert "workload" in d["config"]
