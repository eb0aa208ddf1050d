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
