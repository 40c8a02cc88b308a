"""agent-react: a ReAct loop. Each turn the model either calls a tool (grammar-constrained JSON,
executed through an MCP server) or finishes; tool results are appended to the same context, so
the conversation's KV is never recomputed. Counterpart of inferlets/agent-react/src/lib.rs."""
import json

from pie_b200.sdk import Context, Ebnf, mcp
from pie_b200.runtime.instruct import Instruct

from ._common import load_model, make_sampler

NAME = "agent-react"


async def main(args):
    args = args or {}
    model = load_model(args)
    server, max_turns = args.get("server", "tools"), int(args.get("max_turns", 3))
    tools = await mcp.list_tools(server)
    ins = model.instruct or Instruct()
    finish = {"name": "finish", "parameters": {"type": "object", "properties": {"answer": {"type": "string", "maxLength": 32}},
                                               "required": ["answer"]}}
    grammar = Ebnf(ins.tool_grammar(list(tools) + [finish]))
    ctx = Context(model)
    if "prompt_tokens" in args:
        ctx.append(args["prompt_tokens"])
    else:
        ctx.system(ins.equip(list(tools) + [finish])).user(args.get("prompt", "Use the tools, then finish.")).cue()
    trace = []
    tok = model.tokenizer()
    for turn in range(max_turns):
        text = await ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 160)), constrain=grammar).collect_text()
        call = json.loads(text)
        if call["name"] == "finish":
            trace.append({"finish": call["arguments"]})
            break
        result = await mcp.call_tool(server, call["name"], call.get("arguments", {}))
        trace.append({"call": call, "result": result})
        ctx.append(tok.encode(ins.answer(call["name"], json.dumps(result))))
        ctx.cue()
    ctx.release()
    return json.dumps({"turns": len(trace), "trace": trace})
