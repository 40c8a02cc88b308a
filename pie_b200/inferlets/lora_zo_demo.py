"""marketing-tab3-lora-spec (adapter part): create a LoRA adapter, nudge it with a few
zeroth-order (evolution-strategies) steps towards a target continuation, and compare greedy
output with and without it. Counterpart of inferlets/marketing-tab3-lora-spec (adapters + ZO)."""
import json

from pie_b200.sdk import Adapter, Logprobs, Sampler

from ._common import load_model, prefill_shared, prompt_context

NAME = "marketing-tab3-lora-spec"


async def score(base, last, target, adapter):
    """Log-probability of `target` after the prompt under the adapter (one teacher-forced pass)."""
    ctx = base.fork()
    seq = last + target
    fwd = ctx.forward().input(seq)
    if adapter is not None:
        fwd.adapter(adapter)
    hs = [fwd.probe(j, Logprobs([seq[j + 1]])) for j in range(len(seq) - 1)]
    out = await fwd.execute()
    ctx.release()
    return sum(out.logprobs(h)[0] for h in hs)


async def main(args):
    args = args or {}
    model = load_model(args)
    base = prompt_context(model, args)
    last = await prefill_shared(base)
    target = [int(t) for t in args.get("target_tokens", [7, 7, 7, 7])]
    ad = Adapter.create(model, rank=int(args.get("rank", 4)), alpha=float(args.get("alpha", 8.0)))
    ad.zo_init(float(args.get("sigma", 0.02)))
    before = await score(base, last, target, ad)
    pop, steps = int(args.get("population", 4)), int(args.get("steps", 3))
    for s in range(steps):
        seeds = [1000 * (s + 1) + i for i in range(pop)]
        scores = []
        for sd in seeds:
            ad.zo_perturb(sd, +1.0)
            scores.append(await score(base, last, target, ad))
            ad.zo_perturb(sd, -1.0)
        ad.zo_update(seeds, scores, lr=float(args.get("lr", 0.05)))
    after = await score(base, last, target, ad)
    plain = await base.fork().append(last).generate(Sampler.argmax(), max_tokens=6).collect_tokens()
    tuned = await base.fork().append(last).generate(Sampler.argmax(), max_tokens=6, adapter=ad).collect_tokens()
    if args.get("save"):
        ad.save(args["save"])
    base.release()
    return json.dumps({"score_before": before, "score_after": after, "plain": plain, "tuned": tuned})
