"""The benchmark's CPU arm (`bench.py --impl reference`): runs without a GPU, loads no CUDA library and
prints one JSON line with the keys the two arms share."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_prints_the_shared_line():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    done = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                          cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    line = json.loads(done.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    assert line["metric"] == "nvfp4_moe_layer_tflops" and line["unit"] == "TFLOP/s" and line["higher_is_better"] is True
    assert line["n_gpus"] == 1 and line["steps"] == 1 and line["gpu_launches"] == 0
    assert line["config"]["workload"].startswith("config 4") and line["config"]["tokens"] == 8192
    baseline = line["cpu_baseline"]
    assert baseline["kind"] == "port" and baseline["cores"] >= 1 and baseline["value"] == line["value"] > 0
    assert "tokens per step" in baseline["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert abs(line["ms_per_step"] - baseline["seconds_per_step"] * 1e3) < 1e-6


def test_other_ranks_of_the_reference_arm_do_no_work():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", RANK="1", WORLD_SIZE="2")
    done = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"],
                          cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-2000:]
    assert done.stdout.strip() == ""
