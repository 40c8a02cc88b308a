"""text-completion-bench: the benchmark inferlet. Prefills a prompt of given token ids, decodes
`max_tokens` tokens with the requested sampler and reports per-token timestamps so that the
harness can derive TTFT and inter-token latency. An optional start gate (a session message)
lets the harness release all inferlets at once. Counterpart of
inferlets/text-completion-bench in the reference (start gate over `session`)."""
from __future__ import annotations

import json
import time

from pie_b200.sdk import Context, Model, runtime, session
from .text_completion import make_sampler

NAME = "text-completion-bench"


async def main(args):
    model = Model.load(args.get("model") or runtime.models()[0])
    if args.get("gate"):
        await session.receive()
    t0 = time.perf_counter()
    ctx = Context(model)
    ctx.append(args["prompt_tokens"])
    constrain = None
    if args.get("json_schema") is not None:          # constrained variant: the mask is recomputed every step
        from pie_b200.sdk import JsonSchema
        constrain = JsonSchema(args["json_schema"])
    gen = ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 256)), constrain=constrain).stop([])
    if args.get("per_step") or constrain is not None:
        # inferlet-driven loop: one forward-pass.execute per token
        stamps, n = [], 0
        async for step in gen:
            out = await step.execute()
            n += len(out.tokens)
            stamps.append(time.perf_counter())
    else:
        # plain generation: the runtime's decode cohort runs the loop and stamps each token
        stream = await gen.run_offloaded()
        stamps, n = list(stream.stamps), len(stream.tokens)
    ctx.release()
    return json.dumps({"t0": t0, "stamps": stamps, "n_tokens": n})
