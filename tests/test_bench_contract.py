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


def test_host_buffer_placement_helper(monkeypatch, tmp_path):
    """``cpus_near_gpu``: the GPU's PCI address -> sysfs local_cpulist -> CPU set, cut down to the
    CPUs this process may use; anything missing means "unknown" (None), never an exception, and
    ``near_gpu`` puts the previous affinity back."""
    import builtins
    import types

    sys.path.insert(0, ROOT)
    import bench

    fake_torch = types.SimpleNamespace(cuda=types.SimpleNamespace(get_device_properties=lambda dev: types.SimpleNamespace(
        pci_domain_id=0, pci_bus_id=0x1b, pci_device_id=0)))
    listing = tmp_path / "local_cpulist"
    real_open = builtins.open
    allowed = sorted(os.sched_getaffinity(0))

    def fake_open(path, *a, **k):
        if str(path) == "/sys/bus/pci/devices/0000:1b:00.0/local_cpulist":
            return real_open(listing, *a, **k)
        return real_open(path, *a, **k)

    monkeypatch.setattr(builtins, "open", fake_open)
    listing.write_text(f"{allowed[0]},{allowed[-1]}-{allowed[-1] + 3}\n")
    assert bench.cpus_near_gpu(fake_torch, 0) == {allowed[0], allowed[-1]}
    before = os.sched_getaffinity(0)
    with bench.near_gpu(fake_torch, 0) as placement:
        assert placement.cpus == {allowed[0], allowed[-1]}
        assert os.sched_getaffinity(0) == placement.cpus
    assert os.sched_getaffinity(0) == before
    listing.write_text("100000-100003\n")          # none of them usable here
    assert bench.cpus_near_gpu(fake_torch, 0) is None
    listing.write_text("not a list\n")
    assert bench.cpus_near_gpu(fake_torch, 0) is None
    no_pci = types.SimpleNamespace(cuda=types.SimpleNamespace(get_device_properties=lambda dev: object()))
    assert bench.cpus_near_gpu(no_pci, 0) is None
    with bench.near_gpu(no_pci, 0) as placement:
        assert placement.cpus is None and os.sched_getaffinity(0) == before


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
