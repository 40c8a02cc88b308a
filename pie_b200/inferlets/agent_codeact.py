"""agent-codeact: each step the model emits {"thought", "kind": "code"|"answer", "code", "answer"}
under a JSON-schema constraint. For "code" the host evaluates the expression in a small arithmetic
interpreter (numbers, + - * / % **, parentheses, min/max/abs/round) and feeds the value back as the
next observation; "answer" ends the loop. Counterpart of inferlets/agent-codeact/src/lib.rs (which
evaluates JavaScript with an embedded interpreter)."""
import ast
import json
import operator

from pie_b200.sdk import JsonSchema

from ._common import load_model, make_sampler, prompt_context

NAME = "agent-codeact"

STEP = {"type": "object", "required": ["thought", "kind"], "properties": {
    "thought": {"type": "string", "maxLength": 40}, "kind": {"enum": ["code", "answer"]},
    "code": {"type": "string", "maxLength": 40}, "answer": {"type": "string", "maxLength": 40}}}

_OPS = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.Div: operator.truediv,
        ast.Mod: operator.mod, ast.Pow: operator.pow, ast.USub: operator.neg, ast.FloorDiv: operator.floordiv}
_FUNCS = {"min": min, "max": max, "abs": abs, "round": round}


def evaluate(expr: str):
    """Arithmetic only: no names, attributes, subscripts or calls beyond the four listed functions."""
    def ev(n):
        if isinstance(n, ast.Expression):
            return ev(n.body)
        if isinstance(n, ast.Constant) and isinstance(n.value, (int, float)):
            return n.value
        if isinstance(n, ast.BinOp) and type(n.op) in _OPS:
            a, b = ev(n.left), ev(n.right)
            if isinstance(n.op, ast.Pow) and abs(b) > 64:
                raise ValueError("exponent too large")
            return _OPS[type(n.op)](a, b)
        if isinstance(n, ast.UnaryOp) and type(n.op) in _OPS:
            return _OPS[type(n.op)](ev(n.operand))
        if isinstance(n, ast.Call) and isinstance(n.func, ast.Name) and n.func.id in _FUNCS and not n.keywords:
            return _FUNCS[n.func.id](*[ev(a) for a in n.args])
        raise ValueError("unsupported expression")
    return ev(ast.parse(expr.strip(), mode="eval"))


async def main(args):
    args = args or {}
    model = load_model(args)
    ctx = prompt_context(model, dict(args, system=args.get("system", "Reply with one JSON step at a time.")),
                         "Compute 6 * 7.")
    steps, trace, answer = int(args.get("max_steps", 4)), [], None
    # a small temperature keeps identical contexts from locking into one continuation
    sampler = make_sampler(dict(args, temperature=args.get("temperature", 0.3)))
    for _ in range(steps):
        raw = await ctx.generate(sampler, max_tokens=int(args.get("step_tokens", 96)), constrain=JsonSchema(STEP)).collect_text()
        try:
            step = json.loads(raw)
        except ValueError:
            trace.append({"error": "unparsable step"})
            break
        if step.get("kind") == "answer":
            answer = step.get("answer", "")
            trace.append({"finish": answer})
            break
        try:
            obs = str(evaluate(step.get("code", "")))
        except Exception as e:  # noqa: BLE001
            obs = "error: " + str(e)
        trace.append({"code": step.get("code", ""), "observation": obs})
        ctx.seal().user("Observation: " + obs).cue()
    ctx.release()
    return json.dumps({"answer": answer, "turns": len(trace), "trace": trace})
