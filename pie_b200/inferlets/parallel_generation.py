"""parallel-generation: fill a shared prompt once, fork it, and decode several continuations
concurrently (they batch together on the device and share the prompt's KV pages).
Counterpart of inferlets/parallel-generation/src/lib.rs."""
import asyncio
import json

from ._common import load_model, make_sampler, prefill_shared, prompt_context

NAME = "parallel-generation"


async def main(args):
    args = args or {}
    model = load_model(args)
    n = int(args.get("n", 4))
    base = prompt_context(model, args, "Give me a fun fact.")
    last = await prefill_shared(base)
    branches = [base.fork().append(last) for _ in range(n)]

    async def run(i, ctx):
        a = dict(args, seed=int(args.get("seed", 1)) + i, temperature=args.get("temperature", 0.8))
        toks = await ctx.generate(make_sampler(a), max_tokens=int(args.get("max_tokens", 32))).collect_tokens()
        ctx.release()
        return toks

    outs = await asyncio.gather(*[run(i, c) for i, c in enumerate(branches)])
    base.release()
    tok = model.tokenizer()
    return json.dumps({"texts": [tok.decode(o) for o in outs], "tokens": outs})
