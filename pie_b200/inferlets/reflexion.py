"""reflexion: retry with verbal memory. Each attempt is checked by a deterministic evaluator
(required length, forbidden tokens); the violations of a failed attempt become a short written
lesson that is prepended to the next attempt, instead of a blind resample. Attempts fork one shared
prompt. Counterpart of inferlets/reflexion/src/lib.rs."""
import json

from ._common import load_model, make_sampler, prefill_shared, prompt_context, strip_stop

NAME = "reflexion"


def evaluate(tokens, min_len, forbidden):
    problems = []
    if len(tokens) < min_len:
        problems.append(f"too short ({len(tokens)} < {min_len})")
    bad = sorted(set(tokens) & set(forbidden))
    if bad:
        problems.append("used forbidden tokens " + ",".join(map(str, bad[:4])))
    return problems


async def main(args):
    args = args or {}
    model = load_model(args)
    tok = model.tokenizer()
    attempts, max_tokens = int(args.get("attempts", 3)), int(args.get("max_tokens", 12))
    min_len, forbidden = int(args.get("min_len", 4)), list(args.get("forbidden_tokens", []))
    root = prompt_context(model, args, "Answer the question.")
    last = await prefill_shared(root)
    lessons, history = [], []
    answer = []
    for a in range(attempts):
        ctx = root.fork().append(last)
        if lessons:
            ctx.append(tok.encode(" Lessons: " + "; ".join(lessons) + ". Try again: "))
        toks = strip_stop(model, await ctx.generate(make_sampler(dict(args, seed=1 + a)), max_tokens=max_tokens)
                          .collect_tokens())
        ctx.release()
        problems = evaluate(toks, min_len, forbidden)
        history.append({"attempt": a, "tokens": toks, "problems": problems})
        answer = toks
        if not problems:
            break
        lessons.append(f"attempt {a + 1} was " + " and ".join(problems))
    root.release()
    return json.dumps({"tokens": answer, "attempts": len(history), "solved": not history[-1]["problems"],
                       "lessons": lessons, "history": history})
