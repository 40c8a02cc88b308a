"""prefix-tree: a two-level tree of prompts; every node's KV is computed once and shared by its
descendants through `fork`. Counterpart of inferlets/prefix-tree/src/lib.rs."""
import asyncio
import json

from pie_b200.sdk import Context

from ._common import load_model, make_sampler

NAME = "prefix-tree"


async def main(args):
    args = args or {}
    model = load_model(args)
    tok = model.tokenizer()
    root_text = args.get("root", "You are a travel guide. ")
    mids = args.get("branches", ["Describe Paris. ", "Describe Kyoto. "])
    leaves = args.get("leaves", ["Focus on food.", "Focus on museums."])
    max_tokens = int(args.get("max_tokens", 16))
    root = Context(model)
    root.append(tok.encode(root_text))
    await root.flush()
    results = {}

    async def leaf(mid_ctx, mid, text):
        ctx = mid_ctx.fork()
        ctx.append(tok.encode(text))
        out = await ctx.generate(make_sampler(args), max_tokens=max_tokens).collect_text()
        ctx.release()
        results[f"{mid}|{text}"] = out

    async def mid(text):
        ctx = root.fork()
        ctx.append(tok.encode(text))
        await ctx.flush()
        await asyncio.gather(*[leaf(ctx, text, l) for l in leaves])
        ctx.release()

    await asyncio.gather(*[mid(m) for m in mids])
    shared = root.committed_page_count()
    root.release()
    return json.dumps({"results": results, "root_committed_pages": shared})
