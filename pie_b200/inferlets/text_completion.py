"""text-completion: fill a prompt, decode up to `max_tokens` tokens, return the text.

Input keys: prompt (str) or prompt_tokens (list[int]), max_tokens, temperature, top_p, top_k,
stop_tokens, return_tokens. Counterpart of inferlets/text-completion/src/lib.rs.
"""
from __future__ import annotations

import json

from pie_b200.sdk import Context, Model, Sampler, runtime

NAME = "text-completion"


def make_sampler(a: dict) -> Sampler:
    t = float(a.get("temperature", 0.0))
    seed = int(a.get("seed", 0))
    if t <= 0:
        return Sampler.argmax()
    if "top_k" in a and "top_p" in a:
        return Sampler.top_k_top_p(t, int(a["top_k"]), float(a["top_p"]), seed)
    if "top_k" in a:
        return Sampler.top_k(t, int(a["top_k"]), seed)
    if "top_p" in a:
        return Sampler.top_p(t, float(a["top_p"]), seed)
    if "min_p" in a:
        return Sampler.min_p(t, float(a["min_p"]), seed)
    return Sampler.multinomial(t, seed)


async def main(args):
    args = args or {}
    model = Model.load(args.get("model") or runtime.models()[0])
    ctx = Context(model)
    if "prompt_tokens" in args:
        ctx.append(args["prompt_tokens"])
    else:
        if args.get("system"):
            ctx.system(args["system"])
        ctx.user(args.get("prompt", "Hello")).cue()
    gen = ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 64)))
    if "stop_tokens" in args:
        gen.stop(args["stop_tokens"])
    if args.get("per_step"):
        # inferlet-driven loop (one forward-pass.execute per token) instead of the runtime's cohort
        async for step in gen:
            await step.execute()
        tokens = list(gen._generated)
    else:
        tokens = await gen.collect_tokens()
    ctx.release()
    if args.get("return_tokens") or "prompt_tokens" in args:
        return json.dumps({"tokens": tokens})
    return model.tokenizer().decode(tokens)
