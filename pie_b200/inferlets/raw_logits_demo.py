"""raw-logits-demo: read the full logit vector of the next token and report its top entries.
Counterpart of inferlets/raw-logits-demo/src/lib.rs."""
import json

import numpy as np

from pie_b200.sdk import Logits

from ._common import load_model, prompt_context

NAME = "raw-logits-demo"


async def main(args):
    args = args or {}
    model = load_model(args)
    ctx = prompt_context(model, args)
    toks, ctx._buffer = ctx.buffer, []
    fwd = ctx.forward().input(toks)
    h = fwd.probe(len(toks) - 1, Logits())
    out = await fwd.execute()
    logits = np.frombuffer(out.logits(h), dtype=np.float32)
    top = np.argsort(logits)[::-1][: int(args.get("k", 5))]
    ctx.release()
    return json.dumps({"vocab": int(logits.shape[0]), "top": [[int(i), float(logits[i])] for i in top]})
