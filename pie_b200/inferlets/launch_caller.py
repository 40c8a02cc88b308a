"""launch-caller: spawn child inferlets with runtime.launch and gather their results.
Counterpart of inferlets/launch-caller/src/lib.rs."""
import asyncio
import json

from pie_b200.sdk import runtime

NAME = "launch-caller"


async def main(args):
    args = args or {}
    texts = args.get("texts", ["alpha", "beta", "gamma"])
    children = [runtime.launch(args.get("callee", "launch-callee"), {"text": t}) for t in texts]
    results = await asyncio.gather(*[c.wait() for c in children])
    return json.dumps({"results": list(results)})
