"""tree-of-thought: breadth-first search over partial solutions. Each level forks every kept
node `branching` ways, samples a short "thought" per fork, scores each thought with the model's
own mean log-probability of it, and keeps the best `beam` nodes. All nodes share their common
prefix pages. Counterpart of inferlets/tree-of-thought/src/lib.rs."""
import asyncio
import json

from pie_b200.sdk import Logprobs

from ._common import load_model, make_sampler, prefill_shared, prompt_context

NAME = "tree-of-thought"


async def expand(node_ctx, last, args, seed, thought_tokens):
    ctx = node_ctx.fork().append(last)
    a = dict(args, seed=seed, temperature=args.get("temperature", 0.9))
    toks = await ctx.generate(make_sampler(a), max_tokens=thought_tokens).stop([]).collect_tokens()
    # score: teacher-forced log-probability of the thought under the node
    sc = node_ctx.fork()
    seq = last + toks
    fwd = sc.forward().input(seq)
    hs = [fwd.probe(j, Logprobs([seq[j + 1]])) for j in range(len(seq) - 1)]
    out = await fwd.execute()
    sc.release()
    score = sum(out.logprobs(h)[0] for h in hs) / max(1, len(hs))
    return ctx, toks, score


async def main(args):
    args = args or {}
    model = load_model(args)
    depth, branching, beam = int(args.get("depth", 2)), int(args.get("branching", 3)), int(args.get("beam", 2))
    thought_tokens = int(args.get("thought_tokens", 6))
    root = prompt_context(model, args, "Solve step by step.")
    last = await prefill_shared(root)
    frontier = [(root, last, [], 0.0)]           # (context without its last token, last token, path, score)
    seed = int(args.get("seed", 1))
    for level in range(depth):
        jobs = []
        for ctx, lst, path, sc in frontier:
            for b in range(branching):
                seed += 1
                jobs.append((path, sc, expand(ctx, lst, args, seed, thought_tokens)))
        results = await asyncio.gather(*[j[2] for j in jobs])
        cands = []
        for (path, sc, _), (cctx, toks, s) in zip(jobs, results):
            cands.append((cctx, toks, path + [toks], sc + s))
        cands.sort(key=lambda c: -c[3])
        for c in cands[beam:]:
            c[0].release()
        for ctx, _, _, _ in frontier:
            if ctx is not root:
                ctx.release()
        # a kept child continues from its own context: hold back its last generated token
        frontier = [(c, await _tail(c), p, s) for c, _, p, s in cands[:beam]]
    best = max(frontier, key=lambda f: f[3])
    tok = model.tokenizer()
    out = {"best_score": best[3], "best_path": [tok.decode(t) for t in best[2]], "levels": depth,
           "nodes_expanded": sum(branching * min(beam, branching ** l) for l in range(depth))}
    for ctx, _, _, _ in frontier:
        ctx.release()
    root.release()
    return json.dumps(out)


async def _tail(ctx):
    """Make `ctx` forkable mid-generation: its last sampled token is pending in the buffer."""
    buf = ctx.buffer
    if buf:
        ctx._buffer = buf[:-1]
        await ctx.flush()
        return buf[-1:]
    return []
