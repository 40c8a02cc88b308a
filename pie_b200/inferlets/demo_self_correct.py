"""demo-self-correct (reflexion): draft an answer, ask the model to critique it on a fork, then
revise on another fork that sees draft and critique. Counterpart of inferlets/demo-self-correct
and inferlets/reflexion."""
import json

from ._common import load_model, make_sampler, prompt_context

NAME = "demo-self-correct"


async def main(args):
    args = args or {}
    model = load_model(args)
    n = int(args.get("max_tokens", 12))
    base = prompt_context(model, args, "What is 17 * 23?")
    draft_ctx = base.fork()
    draft = await draft_ctx.generate(make_sampler(args), max_tokens=n).collect_text()
    crit_ctx = draft_ctx.fork()
    crit_ctx.user("Point out any mistake in the answer above.").cue()
    critique = await crit_ctx.generate(make_sampler(args), max_tokens=n).collect_text()
    fix_ctx = crit_ctx.fork()
    fix_ctx.user("Give the corrected final answer.").cue()
    final = await fix_ctx.generate(make_sampler(args), max_tokens=n).collect_text()
    for c in (fix_ctx, crit_ctx, draft_ctx, base):
        c.release()
    return json.dumps({"draft": draft, "critique": critique, "final": final})
