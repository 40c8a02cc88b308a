"""template-generation: fill the holes of a text template; each hole is generated under its own
regular expression while the fixed text between holes is appended as is, all in one context.
Counterpart of inferlets/template-generation/src/lib.rs."""
import json

from pie_b200.sdk import Regex

from ._common import load_model, make_sampler, prompt_context

NAME = "template-generation"

DEFAULT = [("Name: ", r"[A-Z][a-z]{2,8}"), ("\nAge: ", r"[1-9][0-9]?"), ("\nMember: ", r"(yes|no)")]


async def main(args):
    args = args or {}
    model = load_model(args)
    tok = model.tokenizer()
    parts = [tuple(p) for p in args.get("template", DEFAULT)]
    ctx = prompt_context(model, args, "Fill in the form.")
    filled, text = {}, ""
    for label, pattern in parts:
        ctx.append(tok.encode(label))
        value = await ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 24)),
                                   constrain=Regex(pattern)).collect_text()
        filled[label.strip().rstrip(":")] = value
        text += label + value
    ctx.release()
    return json.dumps({"text": text, "fields": filled})
