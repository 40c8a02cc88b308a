"""Helpers shared by the example inferlets."""
from __future__ import annotations

from pie_b200.sdk import Context, Model, runtime

from .text_completion import make_sampler  # noqa: F401  (re-exported)


def load_model(args: dict) -> Model:
    return Model.load((args or {}).get("model") or runtime.models()[0])


def prompt_context(model: Model, args: dict, default: str = "Hello") -> Context:
    """A context holding the request's prompt (raw tokens, or chat-formatted text), not yet flushed."""
    ctx = Context(model)
    if "prompt_tokens" in args:
        ctx.append(args["prompt_tokens"])
    else:
        if args.get("system"):
            ctx.system(args["system"])
        ctx.user(args.get("prompt", default)).cue()
    return ctx


def strip_stop(model: Model, tokens):
    stop = set(model.tokenizer().eos_tokens)
    out = list(tokens)
    while out and out[-1] in stop:
        out.pop()
    return out


async def prefill_shared(ctx: Context):
    """Run all but the last pending token through the model and return that last token: forks of
    `ctx` then share the prompt's KV pages and each samples its own first token from `last`."""
    buf = ctx.buffer
    head, last = buf[:-1], buf[-1:]
    ctx._buffer = head
    await ctx.flush()
    return last
