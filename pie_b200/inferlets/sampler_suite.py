"""sampler-suite: one step with every sampler and probe the API offers, on forks of one prompt.
Counterpart of inferlets/sampler-suite/src/lib.rs."""
import json

import numpy as np

from pie_b200.sdk import Distribution, Entropy, Logits, Logprob, Logprobs, Sampler

from ._common import load_model, prefill_shared, prompt_context

NAME = "sampler-suite"


async def main(args):
    args = args or {}
    model = load_model(args)
    base = prompt_context(model, args)
    last = await prefill_shared(base)
    ctx = base.fork()
    fwd = ctx.forward().input(last)
    samplers = {"argmax": Sampler.argmax(), "multinomial": Sampler.multinomial(1.0, 7),
                "top_k": Sampler.top_k(0.8, 20, 7), "top_p": Sampler.top_p(0.8, 0.9, 7),
                "min_p": Sampler.min_p(0.8, 0.05, 7), "top_k_top_p": Sampler.top_k_top_p(0.8, 20, 0.9, 7)}
    hs = {k: fwd.sample([0], s) for k, s in samplers.items()}
    h_dist = fwd.probe(0, Distribution(1.0, 5))
    h_logits = fwd.probe(0, Logits())
    h_ent = fwd.probe(0, Entropy())
    out = await fwd.execute()
    res = {k: out.token(h) for k, h in hs.items()}
    ids, probs = out.distribution(h_dist)
    logits = np.frombuffer(out.logits(h_logits), dtype=np.float32)
    res["dist_top5"] = list(zip([int(i) for i in ids], [float(p) for p in probs]))
    res["logits_argmax"] = int(logits.argmax())
    res["entropy"] = out.entropy(h_ent)
    # log-probability of the arg-max token, asked for in a second pass on another fork
    ctx2 = base.fork()
    fwd2 = ctx2.forward().input(last)
    h_lp = fwd2.probe(0, Logprob(res["argmax"]))
    h_lps = fwd2.probe(0, Logprobs([res["argmax"], res["multinomial"]]))
    out2 = await fwd2.execute()
    res["logprob_argmax"] = out2.logprobs(h_lp)[0]
    res["logprobs"] = out2.logprobs(h_lps)
    for c in (ctx, ctx2, base):
        c.release()
    return json.dumps(res)
