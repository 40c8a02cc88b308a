"""Determinism ledger: greedy (temperature 0) output of the example workloads on the tiny presets,
hashed and compared with a committed ledger, so that a refactor that changes a single token shows.

    python -m pie_b200.bench.determinism            # compare with determinism_ledger.json
    python -m pie_b200.bench.determinism --update   # rewrite the ledger (after an intended change)

Each case runs through the whole engine on the CPU driver in fp32 (inferlet -> scheduler -> paged
driver), twice, and must also agree with itself. Counterpart of the reference's
benches/smoke_deterministic.py + smoke_deterministic_ledger.json (sha of temp-0 output per model).
"""
from __future__ import annotations

import argparse
import hashlib
import json
from pathlib import Path

import numpy as np
import torch

LEDGER = Path(__file__).with_name("determinism_ledger.json")

CASES = [
    ("tiny-llama", "text-completion", {"max_tokens": 24}),
    ("tiny-llama", "parallel-generation", {"n": 3, "max_tokens": 8, "temperature": 0.0}),
    ("tiny-llama", "jacobi-decoding", {"window": 4, "max_tokens": 16}),
    ("tiny-qwen3-moe", "text-completion", {"max_tokens": 16}),
    ("tiny-gpt-oss", "text-completion", {"max_tokens": 16}),
    ("tiny-olmo2", "text-completion", {"max_tokens": 16}),
]


def run_case(preset_name: str, program: str, args: dict) -> str:
    from ..driver.executor import TorchDriver
    from ..inferlets import install_all
    from ..models.config import preset
    from ..models.weights import random_weights
    from ..runtime.engine import Engine, EngineConfig
    cfg = preset(preset_name)
    w = random_weights(cfg, "cpu", torch.float32, seed=0)
    drv = TorchDriver(cfg, device="cpu", weights=w, num_pages=128, page_size=16, max_requests=16, max_tokens=256)
    eng = Engine(EngineConfig())
    from ..runtime.tokenizer import ByteTokenizer
    eng.add_model(cfg.name, drv, tokenizer=ByteTokenizer(cfg.vocab_size))
    install_all(eng)
    try:
        prompt = np.random.default_rng(1).integers(0, cfg.vocab_size, 32).tolist()
        out = json.loads(eng.run(program, dict(args, prompt_tokens=prompt, stop_tokens=[]), timeout=600))
    finally:
        eng.shutdown()
    return hashlib.sha256(json.dumps(out["tokens"], separators=(",", ":")).encode()).hexdigest()


def run_all() -> dict:
    out = {}
    for preset_name, program, args in CASES:
        a, b = run_case(preset_name, program, args), run_case(preset_name, program, args)
        if a != b:
            raise AssertionError(f"{preset_name}/{program}: two runs disagree")
        out[f"{preset_name}/{program}"] = a
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--update", action="store_true")
    a = ap.parse_args()
    got = run_all()
    if a.update or not LEDGER.exists():
        LEDGER.write_text(json.dumps({"torch": torch.__version__, "cases": got}, indent=1) + "\n")
        print(f"ledger written: {len(got)} cases")
        return 0
    want = json.loads(LEDGER.read_text())["cases"]
    bad = [k for k in got if want.get(k) != got[k]]
    for k in got:
        print(("MISMATCH " if k in bad else "ok       ") + k)
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
