"""watermarking: green-list watermark (Kirchenbauer et al.) done in the inferlet: each step reads
the raw logits, adds `delta` to a pseudo-random half of the vocabulary keyed by the previous
token, and samples on the host. Returns the tokens and the detection z-score.
Counterpart of inferlets/watermarking/src/lib.rs."""
import json
import math

import numpy as np

from pie_b200.sdk import Logits

from ._common import load_model, prompt_context

NAME = "watermarking"


def green_list(prev_token: int, vocab: int, gamma: float, key: int) -> np.ndarray:
    rng = np.random.default_rng((prev_token * 1000003 + key) & 0x7FFFFFFF)
    return rng.random(vocab) < gamma


def z_score(tokens, prompt_last: int, vocab: int, gamma: float, key: int) -> float:
    prev, hits = prompt_last, 0
    for t in tokens:
        hits += bool(green_list(prev, vocab, gamma, key)[t])
        prev = t
    n = max(1, len(tokens))
    return (hits - gamma * n) / math.sqrt(n * gamma * (1 - gamma))


async def main(args):
    args = args or {}
    model = load_model(args)
    gamma, delta, key = float(args.get("gamma", 0.5)), float(args.get("delta", 4.0)), int(args.get("key", 42))
    temperature = float(args.get("temperature", 1.0))
    ctx = prompt_context(model, args)
    pending, ctx._buffer = ctx.buffer, []
    first_prev = pending[-1]
    rng = np.random.default_rng(int(args.get("seed", 0)))
    tokens = []
    for _ in range(int(args.get("max_tokens", 32))):
        fwd = ctx.forward().input(pending)
        h = fwd.probe(len(pending) - 1, Logits())
        out = await fwd.execute()
        logits = np.frombuffer(out.logits(h), dtype=np.float32).astype(np.float64)
        logits = logits + delta * green_list(pending[-1], logits.shape[0], gamma, key)
        p = np.exp((logits - logits.max()) / max(temperature, 1e-6))
        p /= p.sum()
        t = int(rng.choice(p.shape[0], p=p))
        tokens.append(t)
        pending = [t]
    vocab = logits.shape[0]
    ctx.release()
    return json.dumps({"tokens": tokens, "z": z_score(tokens, first_prev, vocab, gamma, key)})
