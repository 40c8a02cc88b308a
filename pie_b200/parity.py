"""Parity harness: run a token sequence through the driver (paged path) and dump the last-token
logits, optionally after a decode step that follows the prefill, for comparison with another
implementation or an earlier build.

    python -m pie_b200.parity --model tiny-llama --tokens 1,2,3,4 --out logits.npy [--device cpu]
        [--decode-after-prefill] [--compare other.npy]
    python -m pie_b200.parity --path CKPT --tokens 1,2,3,4 --hf --out hf.npy     # the same row from Hugging Face
                                                                                    # transformers (fp32, eager attention)

Counterpart of driver/cuda/src/parity_harness.cpp (--parity-tokens / --parity-out /
--parity-paged / --parity-decode-after-prefill; driver/cuda/src/entry.cpp:123-138).
"""
from __future__ import annotations

import argparse
import json

import numpy as np


def run(model: str, tokens, device: str = "cpu", path: str = "", decode_after_prefill: bool = False, seed: int = 0):
    import torch
    from .driver.executor import TorchDriver
    from .driver.schema import SamplerKind, SamplerSpec
    from .models.config import ModelConfig, preset
    from .runtime.scheduler import PendingRequest, fold

    weights = None
    if path:
        from .models import loader
        cfg, weights = loader.load_checkpoint(path, device, dtype="float32" if device == "cpu" else None)
    else:
        cfg = preset(model)
    drv = TorchDriver(cfg, device, weights=weights, num_pages=max(8, len(tokens) // 16 + 4), page_size=16,
                      max_requests=4, max_tokens=max(256, len(tokens) + 8), seed=seed)
    raw = SamplerSpec(SamplerKind.RAW_LOGITS)
    pages = list(range(len(tokens) // 16 + 2))
    if decode_after_prefill:
        head, last = tokens[:-1], tokens[-1]
        drv.fire_batch(fold([PendingRequest(0, head, list(range(len(head))), pages, 0, [])], 16))
        resp = drv.fire_batch(fold([PendingRequest(0, [last], [len(head)], pages, len(head), [(0, raw)])], 16))
    else:
        resp = drv.fire_batch(fold([PendingRequest(0, list(tokens), list(range(len(tokens))), pages, 0,
                                                   [(len(tokens) - 1, raw)])], 16))
    return np.frombuffer(resp.slots[0].logits, dtype=np.float32).copy()


def run_hf(path: str, tokens) -> np.ndarray:
    """Last-token logits of the checkpoint at `path` from Hugging Face transformers (the HF parity dumper of the
    reference's `scripts/`): fp32 on the host, eager attention, no cache."""
    import torch
    from transformers import AutoModelForCausalLM
    m = AutoModelForCausalLM.from_pretrained(path, dtype=torch.float32, attn_implementation="eager")
    m.eval()
    with torch.no_grad():
        return m(torch.tensor([list(tokens)])).logits[0, -1].float().numpy().copy()


def compare(a: np.ndarray, b: np.ndarray) -> dict:
    cos = float(np.dot(a, b) / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-12))
    return {"cos": cos, "max_abs": float(np.abs(a - b).max()), "argmax_equal": bool(a.argmax() == b.argmax()),
            "top5_overlap": len(set(np.argsort(a)[-5:]) & set(np.argsort(b)[-5:]))}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny-llama")
    ap.add_argument("--path", default="", help="checkpoint directory (safetensors + config.json)")
    ap.add_argument("--tokens", required=True, help="comma-separated token ids")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--out", default="")
    ap.add_argument("--decode-after-prefill", action="store_true")
    ap.add_argument("--compare", default="")
    ap.add_argument("--hf", action="store_true", help="dump from Hugging Face transformers instead of the driver")
    a = ap.parse_args()
    toks = [int(t) for t in a.tokens.split(",") if t.strip()]
    logits = run_hf(a.path, toks) if a.hf else run(a.model, toks, a.device, a.path, a.decode_after_prefill)
    if a.out:
        np.save(a.out, logits)
    rep = {"vocab": int(logits.shape[0]), "argmax": int(logits.argmax()), "max": float(logits.max())}
    if a.compare:
        rep.update(compare(logits, np.load(a.compare)))
    print(json.dumps(rep))


if __name__ == "__main__":
    main()
