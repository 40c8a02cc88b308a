"""agentic-fork: prefill a shared prefix once, fork its KV pages `branches` ways, decode
`tokens` tokens per branch with per-branch seeded top-k sampling, drop the branches back to the
prefix, and repeat for `rounds` rounds. The prefix pages are computed once and shared by every
branch of every round. The workload shape of parallel-generation / best-of-n agents
(inferlets/parallel-generation/src/lib.rs, inferlets/best-of-n/src/lib.rs:31-80)."""
import asyncio
import json
import time

from pie_b200.sdk import Context, Sampler

from ._common import load_model, prefill_shared

NAME = "agentic-fork"


async def main(args):
    args = args or {}
    model = load_model(args)
    branches, tokens, rounds = int(args.get("branches", 8)), int(args.get("tokens", 128)), int(args.get("rounds", 4))
    top_k, temperature, seed0 = int(args.get("top_k", 50)), float(args.get("temperature", 1.0)), int(args.get("seed", 1))
    t0 = time.perf_counter()
    base = Context(model)
    base.append(args["prefix_tokens"])
    last = await prefill_shared(base)
    t_prefill = time.perf_counter() - t0
    produced, stamps = 0, []

    async def branch(r, b):
        ctx = base.fork().append(last)
        gen = ctx.generate(Sampler.top_k(temperature, top_k, seed0 + 1000 * r + b), max_tokens=tokens).stop([])
        toks = await gen.collect_tokens()
        ctx.release()                                   # "trim back to the prefix": the branch pages go away
        return len(toks)

    for r in range(rounds):
        counts = await asyncio.gather(*[branch(r, b) for b in range(branches)])
        produced += sum(counts)
        stamps.append(time.perf_counter() - t0)
    shared = base.committed_page_count()
    base.release()
    return json.dumps({"tokens": produced, "prefill_s": t_prefill, "round_ends_s": stamps, "prefix_pages": shared})
