"""jacobi-decoding: fixed-point parallel decoding. A window of guessed tokens is verified in one
pass; the accepted prefix is kept, the rest of the window is refreshed from what the model just
predicted at those positions, and the loop repeats. Greedy output equals plain greedy decoding.
Counterpart of inferlets/jacobi-decoding/src/lib.rs (manual speculation)."""
import json

from pie_b200.sdk import Sampler

from ._common import load_model, prompt_context

NAME = "jacobi-decoding"


async def main(args):
    args = args or {}
    model = load_model(args)
    window, max_tokens = int(args.get("window", 4)), int(args.get("max_tokens", 24))
    ctx = prompt_context(model, args)
    pending, ctx._buffer = ctx.buffer, []
    sampler = Sampler.argmax()
    guess = [0] * window
    tokens, passes = [], 0
    while len(tokens) < max_tokens:
        fwd = ctx.forward().input(pending).speculative(guess)
        last = len(pending) - 1
        h = fwd.sample(list(range(last, last + 1 + len(guess))), sampler)
        out = await fwd.execute()
        pred = out.tokens_at(h)                      # pred[i] = model's token after (pending + guess[:i])
        acc = 0
        while acc < len(guess) and guess[acc] == pred[acc]:
            acc += 1
        new = pred[:acc + 1]
        passes += 1
        tokens.extend(new)
        # the runtime keeps the KV of the accepted prefix only; rejected guesses are overwritten
        pending = new[-1:]
        # next window: the model's own predictions past the accepted point, shifted
        guess = (pred[acc + 1:] + [0] * window)[:window]
    ctx.release()
    return json.dumps({"tokens": tokens[:max_tokens], "passes": passes})
