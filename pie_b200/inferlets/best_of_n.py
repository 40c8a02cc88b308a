"""best-of-n: sample n continuations of one prompt from forks of its context, score each by the
mean log-probability the model gives its own tokens (a probe on every step), return the best.
Counterpart of inferlets/best-of-n/src/lib.rs:31-80."""
import asyncio
import json

from pie_b200.sdk import Logprobs

from ._common import load_model, make_sampler, prefill_shared, prompt_context

NAME = "best-of-n"


async def main(args):
    args = args or {}
    model = load_model(args)
    n = int(args.get("n", 4))
    max_tokens = int(args.get("max_tokens", 24))
    base = prompt_context(model, args, "Write one sentence about the sea.")
    last = await prefill_shared(base)

    async def run(i):
        ctx = base.fork()
        ctx.append(last)
        a = dict(args, seed=int(args.get("seed", 1)) + i, temperature=args.get("temperature", 0.9))
        toks = await ctx.generate(make_sampler(a), max_tokens=max_tokens).collect_tokens()
        ctx.release()
        # teacher-forced scoring pass on another fork: logprob of token j at the row that predicts it
        sc = base.fork()
        seq = last + toks
        fwd = sc.forward().input(seq)
        handles = [fwd.probe(j, Logprobs([seq[j + 1]])) for j in range(len(seq) - 1)]
        out = await fwd.execute()
        lps = [out.logprobs(h)[0] for h in handles]
        sc.release()
        return toks, (sum(lps) / max(1, len(lps)))

    results = await asyncio.gather(*[run(i) for i in range(n)])
    base.release()
    best = max(range(n), key=lambda i: results[i][1])
    tok = model.tokenizer()
    return json.dumps({"best": tok.decode(results[best][0]), "best_index": best,
                       "scores": [r[1] for r in results], "tokens": [r[0] for r in results]})
