"""demo-mcp-tools: discover the tools of an MCP server, let the model emit one grammar-constrained
tool call, execute it through the server and feed the result back for a final answer.
Counterpart of inferlets/demo-mcp-tools and inferlets/mcp-example (MCP client + tool use)."""
import json

from pie_b200.sdk import Context, chat, mcp

from ._common import load_model, make_sampler

NAME = "demo-mcp-tools"


async def main(args):
    args = args or {}
    model = load_model(args)
    server = args.get("server", "tools")
    tools = await mcp.list_tools(server)
    ctx = Context(model)
    if model.instruct is not None:
        ctx.system(chat.equip(model, tools))
    ctx.user(args.get("prompt", "Use a tool."))
    ctx.cue()
    if model.instruct is not None:
        constraint = chat.tool_call_constraint(model, tools)
    else:
        from pie_b200.sdk import Ebnf
        from pie_b200.runtime.instruct import Instruct
        constraint = Ebnf(Instruct().tool_grammar(tools))
    text = await ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 200)),
                              constrain=constraint).collect_text()
    call = json.loads(text)
    result = await mcp.call_tool(server, call["name"], call.get("arguments", {}))
    ctx.release()
    return json.dumps({"call": call, "result": result})
