"""The benchmark's reference arm runs on CPU only: check that it prints one JSON line with the
keys the contract asks for, and that ranks other than 0 stay silent."""
import json
import os
import subprocess
import sys

import pytest

from conftest import ROOT


def _run(env_extra):
    env = dict(os.environ, **env_extra)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr
    return out.stdout.strip()


def test_reference_arm_prints_one_json_line():
    text = _run({"RANK": "0", "WORLD_SIZE": "1"})
    lines = [l for l in text.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference"
    for key in ("metric", "value", "unit", "steps", "warmup", "ms_per_step", "higher_is_better", "dtype", "config",
                "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["value"] > 0 and d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in d["config"]
    # the same configuration as the GPU arm: the full batch, not a sub-sample
    assert d["cpu_baseline"]["sample"].startswith("64 of 64 samples") and d["config"]["global_batch"] == 64


def test_reference_arm_other_ranks_print_nothing():
    assert _run({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}) == ""


@pytest.mark.gpu
@pytest.mark.parametrize("workload", ["c3", "c4"])
def test_training_workloads_print_one_json_line(workload):
    """The forward + backward workloads at a reduced batch: one JSON line with finite gradients."""
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--workload", workload, "--batch", "4",
                          "--steps", "1", "--warmup", "1"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["metric"] == "neuron_updates_per_sec" and d["value"] > 0 and d["config"]["finite"]
    assert d["config"]["forward_ms"] > 0 and d["config"]["backward_ms"] > 0
    assert workload.upper() in d["config"]["workload"] and d["roofline"]["bound"] == "fp32"


@pytest.mark.gpu
def test_headline_line_reports_the_binding_bound():
    """The headline workload alone: the top level of `roofline` is the binding (FP32) bound against a peak measured
    in the same run, the HBM bound is nested, and the traffic figure names the profile it was taken from."""
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--workload", "c2", "--steps", "3",
                          "--no-cpu-baseline"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    r = d["roofline"]
    assert r["bound"] == "fp32" and r["unit"] == "TFLOP/s" and "measured in this run" in r["peak_source"]
    assert 0 < r["frac"] < 1.2 and 40 < r["peak"] < 90 and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
    assert r["other_bound"]["bound"] == "hbm" and r["traffic_source"].startswith("constant from the ncu capture")
    assert d["e2e"]["h2d_bytes_per_step"] > 0 and d["gpu_launches"] > 0 and not d["config"]["device_failure_flag"]


@pytest.mark.gpu
def test_small_workload_graph_replay_equals_launch_by_launch():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--workload", "c1", "--steps", "5"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    d = json.loads(out.stdout.strip().splitlines()[-1])
    assert d["config"]["graph_equals_launch_by_launch"] and not d["config"]["device_failure_flag"]
    assert d["value"] > 0 and d["gpu_launches"] > 0
