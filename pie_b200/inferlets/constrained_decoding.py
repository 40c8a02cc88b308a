"""constrained-decoding: generate text that conforms to a grammar.

Input keys: prompt / prompt_tokens, one of json_schema (object or string), regex, ebnf, or
any_json (true); max_tokens, temperature/top_p/top_k. Returns the generated text (JSON output is
re-serialised compactly when it parses). Counterpart of inferlets/constrained-decoding/src/lib.rs
and inferlets/python-constrained-decoding.
"""
from __future__ import annotations

import json

from pie_b200.sdk import AnyJson, Context, Ebnf, JsonSchema, Model, Regex, runtime

from .text_completion import make_sampler

NAME = "constrained-decoding"


def pick_constraint(args: dict):
    if "json_schema" in args:
        return JsonSchema(args["json_schema"])
    if "regex" in args:
        return Regex(args["regex"])
    if "ebnf" in args:
        return Ebnf(args["ebnf"])
    return AnyJson()


async def main(args):
    args = args or {}
    model = Model.load(args.get("model") or runtime.models()[0])
    ctx = Context(model)
    if "prompt_tokens" in args:
        ctx.append(args["prompt_tokens"])
    else:
        ctx.user(args.get("prompt", "Reply in the requested format.")).cue()
    gen = ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 256)), constrain=pick_constraint(args))
    text = await gen.collect_text()
    ctx.release()
    return text
