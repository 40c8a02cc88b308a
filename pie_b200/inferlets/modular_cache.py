"""modular-cache: prompt modules (a system prompt, tool descriptions, documents) are prefilled once
and saved as named snapshots; a request assembles its context by opening the module that matches its
longest prefix and appending only the rest. Later runs reuse the saved KV without recomputing it.
Counterpart of inferlets/modular-cache-rust (-python, -js)."""
import hashlib
import json

from pie_b200.sdk import Context

from ._common import load_model, make_sampler

NAME = "modular-cache"


def key_of(tokens) -> str:
    return "module-" + hashlib.blake2s(json.dumps(list(tokens)).encode(), digest_size=8).hexdigest()


async def main(args):
    args = args or {}
    model = load_model(args)
    tok = model.tokenizer()
    modules = [m if isinstance(m, list) else tok.encode(m) for m in args.get("modules", ["You are terse. ", "Context: none. "])]
    question = args.get("question_tokens") or tok.encode(args.get("question", "Hi?"))
    if args.get("clear"):
        prefix = []
        for m in modules:
            prefix += m
            try:
                Context.delete(model, key_of(prefix))
            except Exception:  # noqa: BLE001 - nothing saved under that prefix
                pass
        return json.dumps({"cleared": len(modules)})
    # longest saved chain of modules
    ctx, reused, prefix = None, 0, []
    for i in range(len(modules), 0, -1):
        pre = [t for m in modules[:i] for t in m]
        ctx = Context.open(model, key_of(pre))
        if ctx is not None:
            reused, prefix = i, pre
            break
    if ctx is None:
        ctx = Context(model)
    computed = 0
    for i in range(reused, len(modules)):
        ctx.append(modules[i])
        await ctx.flush()
        prefix += modules[i]
        computed += len(modules[i])
        ctx.save(key_of(prefix))                   # every longer prefix becomes reusable as well
    ctx.append(question)
    tokens = await ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 8))).collect_tokens()
    ctx.release()
    return json.dumps({"tokens": tokens, "modules_reused": reused, "module_tokens_computed": computed})
