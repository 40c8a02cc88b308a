"""attention-sink: StreamingLLM-style decoding. Every new token attends to the first `sink` tokens
and to the last `window` tokens only; the mask is a BRLE row [0, sink, gap, window] per input token.
Counterpart of inferlets/attention-sink/src/lib.rs:40-49."""
import json

from ._common import load_model, make_sampler, prompt_context

NAME = "attention-sink"


def sink_mask(kv_len: int, sink: int, window: int):
    """BRLE over kv positions [0, kv_len): true on the first `sink` and the last `window`."""
    if kv_len <= sink + window:
        return [0, kv_len]
    return [0, sink, kv_len - sink - window, window]


async def main(args):
    args = args or {}
    model = load_model(args)
    sink, window = int(args.get("sink", 4)), int(args.get("window", 32))
    max_tokens = int(args.get("max_tokens", 32))
    ctx = prompt_context(model, args, "Tell me a long story.")
    sampler = make_sampler(args)
    pending = ctx.buffer
    ctx._buffer = []
    tokens = []
    while len(tokens) < max_tokens:
        start = ctx.seq_len
        fwd = ctx.forward().input(pending)
        fwd.attention_mask([sink_mask(start + i + 1, sink, window) for i in range(len(pending))])
        h = fwd.sample([len(pending) - 1], sampler)
        out = await fwd.execute()
        t = out.token(h)
        tokens.append(t)
        pending = [t]
        if t in model.tokenizer().eos_tokens:
            break
    ctx.release()
    return json.dumps({"tokens": tokens, "text": model.tokenizer().decode(tokens)})
