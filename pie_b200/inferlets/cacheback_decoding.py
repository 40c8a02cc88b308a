"""cacheback-decoding: speculative decoding with a drafter that lives on its own context. The
drafter greedily proposes `draft_len` tokens; the main context runs them as ordinary inputs in one
pass and reads the model's prediction after each; the agreeing prefix (plus the model's own next
token) is kept and BOTH contexts roll their rejected tail back with `truncate`. Greedy output is
the plain greedy continuation. Counterpart of inferlets/cacheback-decoding/src/lib.rs."""
import json

from pie_b200.sdk import Sampler

from ._common import load_model, prompt_context

NAME = "cacheback-decoding"


async def main(args):
    args = args or {}
    model = load_model(args)
    draft_len, max_tokens = int(args.get("draft_len", 4)), int(args.get("max_tokens", 24))
    main_ctx = prompt_context(model, args)
    prompt = main_ctx.buffer
    drafter = main_ctx.fork()                      # here the drafter is the same model on a second context
    greedy = Sampler.argmax()
    # both contexts hold the prompt except its last token, which is the first pending input
    main_ctx._buffer, drafter._buffer = prompt[:-1], prompt[:-1]
    await main_ctx.flush()
    await drafter.flush()
    pending, tokens, passes, accepted_total = prompt[-1:], [], 0, 0
    while len(tokens) < max_tokens:
        # draft: the drafter decodes draft_len tokens one by one
        drafts, feed = [], list(pending)
        for _ in range(draft_len):
            f = drafter.forward().input(feed)
            h = f.sample([len(feed) - 1], greedy)
            t = (await f.execute()).token(h)
            drafts.append(t)
            feed = [t]
        # verify: pending + drafts as regular inputs of one pass, a sampler after every position
        seq = list(pending) + drafts
        f = main_ctx.forward().input(seq)
        first = len(pending) - 1
        h = f.sample(list(range(first, len(seq))), greedy)
        pred = (await f.execute()).tokens_at(h)     # pred[i]: the model's token after pending + drafts[:i]
        passes += 1
        acc = 0
        while acc < len(drafts) and drafts[acc] == pred[acc]:
            acc += 1
        accepted_total += acc
        tokens.extend(drafts[:acc] + [pred[acc]])
        # roll back what was rejected: the main context ran all drafts, the drafter ran all but the last
        main_ctx.truncate(len(drafts) - acc)
        drafter.truncate(max(0, len(drafts) - 1 - acc))
        if acc == len(drafts):
            # every draft was right: the drafter has not seen its own last draft yet
            pending_d = [drafts[-1], pred[acc]]
        else:
            pending_d = [pred[acc]]
        # the bonus token is the next pending input of both contexts
        pending = [pred[acc]]
        if len(pending_d) == 2:
            f = drafter.forward().input(pending_d[:1])
            await f.execute()
    main_ctx.release()
    drafter.release()
    return json.dumps({"tokens": tokens[:max_tokens], "passes": passes,
                       "mean_accepted": accepted_total / max(1, passes)})
