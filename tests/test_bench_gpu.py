"""The benchmark program on a GPU, both arms, at one layer of the headline shape (seconds, not minutes)."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.slow]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=900)


def test_our_arm_prints_the_contracts_line_and_checks_the_ids_of_the_timed_loop():
    r = run("--layers", "1", "--steps", "40", "--warmup", "3", "--no-points")
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "e2e", "gpu_launches", "prefill", "roofline", "points", "clocks"):
        assert key in line
    assert line["config"]["layers"] == 1 and line["config"]["layers_full"] == 24 and len(line["config"]) <= 20
    assert line["gpu_launches"] > 0 and line["library_gemm_launches"] == 0
    checked = line["e2e"]["ids_checked"]
    assert checked["steps"] == 32 and checked["equal_first_8"] * 2 >= checked["of"] == 8
    assert line["roofline"]["bound"] == "hbm" and 0 < line["roofline"]["frac"] < 1.5
    assert line["prefill"]["tokens"] == 2048 and line["prefill"]["first_ms"] > 0


def test_reference_arm_runs_the_references_own_gpu_path():
    r = run("--impl", "reference", "--layers", "1", "--steps", "2", "--warmup", "3", "--batch", "2")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" not in line, line
    assert line["dtype"] == "fp32" and line["value"] > 0 and line["e2e"]["value"] > 0 and line["e2e"]["value"] <= line["value"] * 1.001
    assert line["config"]["layers"] == 1 and line["config"]["global_batch"] == 2 and len(line["config"]) <= 20
    assert line["e2e"]["d2h_bytes_per_step"] == 2 * 151936 * 4
