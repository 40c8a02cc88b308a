"""windowed-attention: sliding-window decoding through per-token attention masks (no sink).
Pages that fall wholly outside the window are dropped from the request by the runtime's page
trim. Counterpart of inferlets/windowed-attention/src/lib.rs."""
import json

from ._common import load_model, make_sampler, prompt_context

NAME = "windowed-attention"


async def main(args):
    args = args or {}
    model = load_model(args)
    window = int(args.get("window", 32))
    max_tokens = int(args.get("max_tokens", 32))
    ctx = prompt_context(model, args, "Tell me a long story.")
    sampler = make_sampler(args)
    pending, ctx._buffer = ctx.buffer, []
    tokens = []
    while len(tokens) < max_tokens:
        start = ctx.seq_len
        fwd = ctx.forward().input(pending)
        rows = []
        for i in range(len(pending)):
            kv = start + i + 1
            rows.append([0, kv] if kv <= window else [kv - window, window])
        fwd.attention_mask(rows)
        h = fwd.sample([len(pending) - 1], sampler)
        t = (await fwd.execute()).token(h)
        tokens.append(t)
        pending = [t]
    ctx.release()
    return json.dumps({"tokens": tokens})
