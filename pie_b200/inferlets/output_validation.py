"""output-validation: sample candidates until one passes a validator (here: a regex), up to
`attempts` tries, each on a fresh fork of the prompt. Counterpart of inferlets/output-validation."""
import json
import re

from ._common import load_model, make_sampler, prefill_shared, prompt_context

NAME = "output-validation"


async def main(args):
    args = args or {}
    model = load_model(args)
    pattern = re.compile(args.get("pattern", r".+"), re.S)
    base = prompt_context(model, args)
    last = await prefill_shared(base)
    tries = []
    for i in range(int(args.get("attempts", 4))):
        ctx = base.fork().append(last)
        a = dict(args, seed=int(args.get("seed", 1)) + i, temperature=args.get("temperature", 0.8))
        text = await ctx.generate(make_sampler(a), max_tokens=int(args.get("max_tokens", 16))).collect_text()
        ctx.release()
        tries.append(text)
        if pattern.fullmatch(text):
            base.release()
            return json.dumps({"ok": True, "text": text, "attempts": i + 1})
    base.release()
    return json.dumps({"ok": False, "text": tries[-1], "attempts": len(tries)})
