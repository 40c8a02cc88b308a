"""demo-parallel-fork: fork one conversation into several follow-up questions answered
concurrently. Counterpart of inferlets/demo-parallel-fork/src/lib.rs."""
import asyncio
import json

from ._common import load_model, make_sampler, prompt_context

NAME = "demo-parallel-fork"


async def main(args):
    args = args or {}
    model = load_model(args)
    base = prompt_context(model, dict(args, prompt=args.get("prompt", "Let us talk about rivers.")))
    await base.flush()
    questions = args.get("questions", ["Which is the longest?", "Which is the widest?", "Which is the deepest?"])

    async def ask(q):
        ctx = base.fork()
        ctx.user(q).cue()
        text = await ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 16))).collect_text()
        ctx.release()
        return text

    answers = await asyncio.gather(*[ask(q) for q in questions])
    base.release()
    return json.dumps(dict(zip(questions, answers)))
