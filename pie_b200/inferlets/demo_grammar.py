"""demo-grammar: decode under a hand-written EBNF grammar (an arithmetic expression).
Counterpart of inferlets/demo-grammar/src/lib.rs."""
from pie_b200.sdk import Ebnf

from ._common import load_model, make_sampler, prompt_context

NAME = "demo-grammar"

EXPR = r'''
root ::= expr
expr ::= term ( [+-] term ){0,3}
term ::= factor ( [*/] factor ){0,2}
factor ::= number | "(" expr ")"
number ::= [1-9] [0-9]{0,2}
'''


async def main(args):
    args = args or {}
    model = load_model(args)
    ctx = prompt_context(model, args, "Write an arithmetic expression.")
    text = await ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 64)),
                              constrain=Ebnf(args.get("ebnf", EXPR))).collect_text()
    ctx.release()
    return text
