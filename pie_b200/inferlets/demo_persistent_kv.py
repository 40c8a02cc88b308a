"""demo-persistent-kv: keep a prompt's KV cache across inferlet runs. The first run fills the
context and saves it under a name; later runs open it (a fork of the saved pages) and continue
without recomputing the prefix. Counterpart of inferlets/demo-persistent-kv/src/lib.rs."""
import json

from pie_b200.sdk import Context

from ._common import load_model, make_sampler

NAME = "demo-persistent-kv"


async def main(args):
    args = args or {}
    model = load_model(args)
    tok = model.tokenizer()
    name = args.get("name", "persistent-demo")
    if args.get("delete"):
        Context.delete(model, name)
        return json.dumps({"deleted": name})
    ctx = Context.open(model, name)
    reused = ctx is not None
    if ctx is None:
        ctx = Context(model)
        ctx.append(tok.encode(args.get("prefix", "The quick brown fox jumps over the lazy dog. " * 4)))
        await ctx.flush()
        ctx.save(name)
    prefix_tokens = ctx.kv_len
    ctx.append(tok.encode(args.get("suffix", " And then")))
    tokens = await ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 16))).collect_tokens()
    ctx.release()
    return json.dumps({"reused": reused, "prefix_tokens": prefix_tokens, "tokens": tokens})
