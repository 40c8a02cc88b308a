"""bench.py contract on a machine without a GPU: the reference arm and the no-CUDA case print one
JSON line and exit 0."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                         timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    return json.loads(lines[0])


def test_reference_arm_reports_unavailable():
    r = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r["impl"] == "reference" and "unavailable" in r and "\n" not in r["unavailable"]


def test_no_cuda_reports_unavailable():
    import torch
    if torch.cuda.is_available():
        return
    r = _run("--steps", "2", "--warmup", "1")
    assert r["value"] is None and r["unavailable"] == "no CUDA device"
