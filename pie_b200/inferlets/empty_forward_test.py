"""empty-forward-test: a forward pass with no input tokens is a no-op that returns no slots.
Counterpart of inferlets/empty-forward-test/src/lib.rs."""
import json

from pie_b200.sdk import Context

from ._common import load_model

NAME = "empty-forward-test"


async def main(args):
    model = load_model(args or {})
    with Context(model) as ctx:
        out = await ctx.forward().execute()
        return json.dumps({"slots": len(out.raw.slots), "seq_len": ctx.seq_len})
