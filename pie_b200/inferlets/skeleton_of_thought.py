"""skeleton-of-thought: first generate a short outline, then expand every outline point in
parallel on forks of the shared context. Counterpart of inferlets/skeleton-of-thought/src/lib.rs."""
import asyncio
import json

from ._common import load_model, make_sampler, prompt_context

NAME = "skeleton-of-thought"


async def main(args):
    args = args or {}
    model = load_model(args)
    tok = model.tokenizer()
    points = int(args.get("points", 3))
    base = prompt_context(model, args, "Explain how a bill becomes law.")
    skeleton = await base.fork().generate(make_sampler(args), max_tokens=int(args.get("skeleton_tokens", 12))).collect_tokens()
    await base.flush()
    chunk = max(1, len(skeleton) // points)
    heads = [skeleton[i * chunk:(i + 1) * chunk] for i in range(points)]

    async def expand(i, head):
        ctx = base.fork()
        ctx.append(tok.encode(f"\nPoint {i + 1}: ") + head)
        text = await ctx.generate(make_sampler(dict(args, seed=i + 1)), max_tokens=int(args.get("point_tokens", 8))).collect_text()
        ctx.release()
        return text

    bodies = await asyncio.gather(*[expand(i, h) for i, h in enumerate(heads)])
    base.release()
    return json.dumps({"skeleton": tok.decode(skeleton), "points": list(bodies)})
