"""The benchmark's reference arm (the C restatement of the reference's CPU arithmetic) runs without a GPU and prints
the line the contract asks for, with the same `config` object the GPU arm prints for that workload."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", *args],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stdout + res.stderr
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    return json.loads(lines[0])


def test_reference_arm_line_for_a_moe_workload():
    sys.path.insert(0, ROOT)
    import argparse
    import bench
    line = _run("--workload", "moe_q4k", "--steps", "1", "--warmup", "1", "--cpu-tokens", "2")
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"):
        assert key in line, key
    assert line["impl"] == "reference" and line["metric"] == bench.MOE_METRIC and line["unit"] == "tokens/s"
    assert line["value"] > 0 and line["gpu_launches"] == 0
    assert line["e2e"]["value"] == line["value"] and line["e2e"]["h2d_bytes_per_step"] == 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    args = argparse.Namespace(workload="moe_q4k", tokens=0, experts=0, act16=False)
    assert line["config"] == bench.moe_config(bench.moe_cfg(args), 1, "strong")


def test_reference_arm_line_for_the_decode_sweep():
    line = _run("--workload", "gemv", "--steps", "1", "--warmup", "1", "--only", "4096x4096")
    assert line["impl"] == "reference" and line["value"] > 0 and line["config"]["workload"]
