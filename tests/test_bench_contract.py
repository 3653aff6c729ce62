"""The JSON line bench.py prints: the reference arm runs on host cores only, so its line can be
checked without a GPU; the keys of our own arm's line are checked on a GPU box."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE_KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
             "scaling", "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches"}


def _run(*args, timeout=900):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], cwd=ROOT,
                         capture_output=True, text=True, timeout=timeout)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_line_on_host_cores():
    d = _run("--impl", "reference", "--steps", "1", "--warmup", "1", "--workload", "cfg2_causal")
    assert BASE_KEYS <= set(d) and d["impl"] == "reference"
    assert d["unit"] == "TFLOPS" and d["higher_is_better"] is True and d["value"] > 0
    assert d["config"]["workload"] == "cfg2_causal"
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["gpu_launches"] == 0


@pytest.mark.gpu
def test_our_arm_line_has_roofline_baseline_e2e_and_clocks():
    d = _run("--steps", "3", "--warmup", "3", "--regions", "3", "--workload", "cfg2_causal")
    assert BASE_KEYS <= set(d) and "impl" not in d
    assert d["n_gpus"] == 1 and d["steps"] == 3 and d["gpu_launches"] == 12
    r = d["roofline"]
    assert r["bound"] == "tensor" and r["unit"] == "TFLOP/s" and 0 < r["frac"] < 1.2
    assert abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9 and r["frac_of_burst_peak"] <= r["frac"]
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["value"] > 0
    assert d["e2e"]["value"] > 0 and d["e2e"]["h2d_bytes_per_step"] > 0
    assert {"sm_mhz", "sm_max_mhz", "reasons"} <= set(d["clocks"])
    assert d["config"]["launch"].startswith("CUDA graph") or d["config"]["launch"].startswith("four")
    assert d["regions"]["count"] == 3 and d["regions"]["min_ms"] <= d["ms_per_step"] <= d["regions"]["max_ms"]
    # (a step of this small workload is replayed from a CUDA graph; the instrumented loop launches
    # its kernels one by one with events between them, so the parts add up to well over the step)
    assert 0.8 < d["kernels"]["sum_of_parts_over_step"] < 3.0
    assert d["kernels"]["from_idle"]["fwd_ms"] > 0 and d["kernels"]["plain_step_ms_right_after"] > 0
    assert "sharded" not in d  # only the default workload carries the sharded configs
