"""raw-completion: continue a raw string without any chat template.
Counterpart of inferlets/raw-completion/src/lib.rs."""
from pie_b200.sdk import Context

from ._common import load_model, make_sampler

NAME = "raw-completion"


async def main(args):
    args = args or {}
    model = load_model(args)
    tok = model.tokenizer()
    with Context(model) as ctx:
        ctx.append(tok.encode(args.get("prompt", "Once upon a time")))
        return await ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 32))).collect_text()
