"""The reference arm of bench.py runs without a GPU: its output contract is checked here (one JSON line on stdout,
the keys the driver reads).  The GPU arm prints the same line plus roofline / clocks; it is checked on a B200."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
COMMON = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
          "dtype", "data", "config", "e2e", "cpu_baseline"}


def run_bench(*args, env=None):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, cwd=ROOT,
                         env=dict(os.environ, **(env or {})), timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    return out.stdout


def test_reference_arm_prints_one_json_line():
    text = run_bench("--impl", "reference", "--steps", "1", "--warmup", "0")
    lines = [l for l in text.splitlines() if l.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert COMMON <= set(line) and line["impl"] == "reference"
    assert line["metric"] == "fused_graph_hbm_gbps" and line["unit"] == "GB/s" and line["higher_is_better"] is True
    assert line["vs_baseline"] is None and line["value"] > 0 and line["steps"] == 1
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in line["config"] and "model" not in line["config"]


def test_reference_arm_other_ranks_exit_quietly():
    assert run_bench("--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0", env={"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}).strip() == ""


@pytest.mark.gpu
def test_gpu_arm_line(tmp_path):
    text = run_bench("--no-extras", "--steps", "5", "--warmup", "3")
    lines = [l for l in text.splitlines() if l.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert COMMON | {"clocks", "gpu_launches", "roofline"} <= set(line)
    # per step: one fused kernel for both graphs, one finalize launch for dg and db
    assert line["gpu_launches"] == 5 * 2 and line["n_gpus"] == 1 and line["dtype"] == "f32"
    r = line["roofline"]
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9 and r["traffic"] > 0
    assert line["e2e"]["h2d_bytes_per_step"] > 0 and line["e2e"]["d2h_bytes_per_step"] > 0 and line["e2e"]["value"] < line["value"]
    assert line["cpu_baseline"]["value"] > 0 and line["value"] / line["cpu_baseline"]["value"] > 100
