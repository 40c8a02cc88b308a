"""demo-custom-spec: hand-rolled speculative decoding with the raw forward API. A fixed draft
(the previous output shifted, "cacheback" style) is attached with `speculative`; the pass returns
the accepted prefix plus one bonus token. Counterpart of inferlets/demo-custom-spec and
inferlets/cacheback-decoding."""
import json

from pie_b200.sdk import Sampler

from ._common import load_model, prompt_context

NAME = "demo-custom-spec"


async def main(args):
    args = args or {}
    model = load_model(args)
    ctx = prompt_context(model, args)
    pending, ctx._buffer = ctx.buffer, []
    max_tokens, depth = int(args.get("max_tokens", 32)), int(args.get("depth", 3))
    sampler = Sampler.argmax()
    history, tokens, passes, accepted_total = list(pending), [], 0, 0
    table = {}                                  # bigram -> next token seen after it
    while len(tokens) < max_tokens:
        draft = []
        key = tuple(history[-2:])
        while len(draft) < depth and key in table:
            draft.append(table[key])
            key = (key[1], draft[-1])
        fwd = ctx.forward().input(pending)
        if draft:
            fwd.speculative(draft)
        last = len(pending) - 1
        h = fwd.sample(list(range(last, last + 1 + len(draft))), sampler)
        out = await fwd.execute()
        sampled = out.tokens_at(h)
        # the walk: draft i is accepted while it equals the token sampled at the row before it
        acc = 0
        while acc < len(draft) and draft[acc] == sampled[acc]:
            acc += 1
        new = sampled[:acc + 1]
        passes += 1
        accepted_total += acc
        for t in new:
            if len(history) >= 2:
                table[tuple(history[-2:])] = t
            history.append(t)
        tokens.extend(new)
        pending = new[-1:]
        # the runtime appended the accepted prefix only; rejected drafts leave no KV behind
    ctx.release()
    return json.dumps({"tokens": tokens[:max_tokens], "passes": passes, "accepted_drafts": accepted_total})
