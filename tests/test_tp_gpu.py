"""Tensor parallelism on real GPUs (needs >= 2): fused peer-memory path and NCCL baseline path
against a single-GPU run of the same weights."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("backend,model", [("fused", "dense"), ("nccl", "dense"), ("fused", "moe"),
                                           ("fused", "moe-ep"), ("nccl", "moe-ep"), ("fused", "dense-fp8"),
                                           ("nccl", "gpt-oss"), ("fused", "gpt-oss"), ("nccl", "olmo2"),
                                           ("nccl", "gemma3"), ("fused", "gemma2"), ("nccl", "qwen2-moe")])
def test_tp2_logits_match_single_gpu(backend, model):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    port = 29511 + ["dense", "moe", "moe-ep", "dense-fp8", "gpt-oss", "olmo2", "gemma3", "gemma2", "qwen2-moe"].index(model) * 2 + (backend == "nccl")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "tp_check.py"), "--backend", backend,
           "--model", model]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert out.returncode == 0 and lines, out.stdout[-2000:] + out.stderr[-4000:]
    rep = json.loads(lines[-1])
    assert rep["ok"], rep
