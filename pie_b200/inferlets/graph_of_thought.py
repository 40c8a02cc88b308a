"""graph-of-thought: `proposals` initial answers are generated concurrently from one shared prompt,
then merged pairwise level by level (each merge prompt quotes its two inputs) until one remains;
a merge starts as soon as its two inputs are ready. Counterpart of inferlets/graph-of-thought/src/lib.rs."""
import asyncio
import json

from ._common import load_model, make_sampler, prefill_shared, prompt_context, strip_stop

NAME = "graph-of-thought"


async def main(args):
    args = args or {}
    model = load_model(args)
    tok = model.tokenizer()
    n, max_tokens = int(args.get("proposals", 4)), int(args.get("max_tokens", 12))
    root = prompt_context(model, args, "Propose a plan.")
    last = await prefill_shared(root)
    merges = 0

    async def propose(i):
        ctx = root.fork().append(last)
        toks = await ctx.generate(make_sampler(dict(args, temperature=args.get("temperature", 0.9), seed=1 + i)),
                                  max_tokens=max_tokens).collect_tokens()
        ctx.release()
        return strip_stop(model, toks)

    async def merge(a, b):
        nonlocal merges
        x, y = await asyncio.gather(a, b)
        merges += 1
        ctx = root.fork().append(last)
        ctx.append(tok.encode(" Option A: ") + x + tok.encode(" Option B: ") + y + tok.encode(" Combined: "))
        toks = await ctx.generate(make_sampler(args), max_tokens=max_tokens).collect_tokens()
        ctx.release()
        return strip_stop(model, toks)

    level = [asyncio.ensure_future(propose(i)) for i in range(n)]
    depth = 0
    while len(level) > 1:
        nxt = [asyncio.ensure_future(merge(level[i], level[i + 1])) for i in range(0, len(level) - 1, 2)]
        if len(level) % 2:
            nxt.append(level[-1])
        level, depth = nxt, depth + 1
    final = await level[0]
    root.release()
    return json.dumps({"tokens": final, "text": tok.decode(final), "merges": merges, "levels": depth})
