"""text-completion-spec: completion with an inferlet-side n-gram speculator; drafts ride along
as extra input tokens and are verified in the same pass.
Counterpart of inferlets/text-completion-spec/src/lib.rs."""
import json

from pie_b200.sdk import NGramSpeculator

from ._common import load_model, make_sampler, prompt_context

NAME = "text-completion-spec"


async def main(args):
    args = args or {}
    model = load_model(args)
    ctx = prompt_context(model, args)
    spec = NGramSpeculator(list(ctx.buffer), n=int(args.get("ngram", 2)), max_draft=int(args.get("max_draft", 4)))
    gen = ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 64)), speculator=spec)
    if "stop_tokens" in args:
        gen.stop(args["stop_tokens"])
    steps = accepted = 0
    async for step in gen:
        out = await step.execute()
        steps += 1
        accepted += max(0, len(out.tokens) - 1)
    tokens = list(gen._generated)
    ctx.release()
    return json.dumps({"tokens": tokens, "steps": steps, "accepted_drafts": accepted})
