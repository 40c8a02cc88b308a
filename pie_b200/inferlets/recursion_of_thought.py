"""recursion-of-thought: divide a problem into independent sub-problems, solve them concurrently on
forks of one shared prefix, and merge the answers on the way back up. The divide step is generated
under a small EBNF grammar ({"parts": ["...", "..."]} or {"leaf": "..."}), so it always parses.
Counterpart of inferlets/recursion-of-thought/src/lib.rs."""
import asyncio
import json

from pie_b200.sdk import Ebnf

from ._common import load_model, make_sampler, prefill_shared, prompt_context

NAME = "recursion-of-thought"

DIVIDE = r'''
root ::= "{\"leaf\":\"" text "\"}" | "{\"parts\":[\"" text "\",\"" text "\"]}"
text ::= [a-zA-Z0-9 ]{1,24}
'''


async def main(args):
    args = args or {}
    model = load_model(args)
    tok = model.tokenizer()
    max_depth, max_tokens = int(args.get("depth", 2)), int(args.get("max_tokens", 48))
    root = prompt_context(model, args, "Solve by splitting into parts.")
    last = await prefill_shared(root)
    calls = {"divide": 0, "leaf": 0, "merge": 0}

    async def solve(task: str, depth: int) -> str:
        ctx = root.fork().append(last).append(tok.encode(" Task: " + task + " Plan: "))
        if depth >= max_depth:
            calls["leaf"] += 1
            text = await ctx.generate(make_sampler(args), max_tokens=8).collect_text()
            ctx.release()
            return text
        calls["divide"] += 1
        raw = await ctx.generate(make_sampler(args), max_tokens=max_tokens, constrain=Ebnf(DIVIDE)).collect_text()
        ctx.release()
        try:
            plan = json.loads(raw)
        except ValueError:
            plan = {"leaf": raw}
        if "leaf" in plan:
            calls["leaf"] += 1
            return plan["leaf"]
        parts = await asyncio.gather(*[solve(p, depth + 1) for p in plan["parts"]])
        calls["merge"] += 1
        m = root.fork().append(last).append(tok.encode(" Combine: " + " | ".join(parts) + " Answer: "))
        text = await m.generate(make_sampler(args), max_tokens=8).collect_text()
        m.release()
        return text

    answer = await solve(args.get("task", "the whole problem"), 0)
    root.release()
    return json.dumps({"answer": answer, **calls})
