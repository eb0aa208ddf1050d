"""The benchmark's reference arm runs without a GPU: its JSON line must carry the keys the driver reads, and the
arm of this library must refuse to run without a CUDA device instead of falling back to anything."""
import json
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parents[1]


def _run(*args):
    return subprocess.run([sys.executable, str(REPO / "bench.py"), *args], capture_output=True, text=True, timeout=300)


def test_reference_arm_prints_the_contract_line():
    res = _run("--impl", "reference", "--workload", "c1", "--steps", "2", "--warmup", "1")
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["higher_is_better"] is True
    assert line["metric"] == "flash-decode HBM GB/s" and line["n_gpus"] == 1 and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "reference" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "C1" in line["config"]["workload"] and "model" not in line["config"]


def test_own_arm_needs_a_gpu():
    import torch

    if torch.cuda.is_available():
        return  # on a GPU box the arm runs; the GPU tests and the driver cover it
    res = _run("--workload", "c1", "--steps", "1", "--warmup", "3", "--no-cpu-baseline")
    assert res.returncode != 0
    assert not any(l.startswith("{") for l in res.stdout.splitlines())   # no result line from a CPU fallback


def test_reference_arm_under_a_launcher_uses_the_host_cores_and_the_global_batch():
    """torch.distributed.run exports OMP_NUM_THREADS=1 and one rank per GPU: rank 0 alone runs the CPU arm, on all
    host cores, over the N per-GPU batches; the other ranks exit 0 without work or output."""
    import os

    env = dict(os.environ, OMP_NUM_THREADS="1", WORLD_SIZE="2", RANK="0", LOCAL_RANK="0")
    cmd = [sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "3"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["n_gpus"] == 2 and line["steps"] == 1 and line["warmup"] == 3
    assert line["config"]["global_batch"] == 32 and "B=16/GPU" in line["config"]["workload"]
    assert line["cpu_baseline"]["cores"] == (os.cpu_count() or 1)
    other = subprocess.run(cmd, capture_output=True, text=True, timeout=120, env=dict(env, RANK="1", LOCAL_RANK="1"))
    assert other.returncode == 0 and other.stdout.strip() == ""
