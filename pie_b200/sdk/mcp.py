"""MCP client for inferlets (WIT `pie:mcp/client`). Tool servers are hosted by a connected client
(`PieClient.register_mcp_server(name, fn)`) or registered in-process on the engine
(`engine.mcp_servers[name] = callable`); the inferlet sends JSON-RPC-shaped requests through the
session that registered the server.

    tools = await mcp.list_tools("calc")
    result = await mcp.call_tool("calc", "add", {"a": 1, "b": 2})

Counterpart of sdk/python/src/inferlet/mcp.py and runtime/src/api/mcp/client.rs.
"""
from __future__ import annotations

import asyncio
import inspect
import json
from typing import Any, List

from . import host


class McpError(RuntimeError):
    pass


async def request(server: str, method: str, params: Any = None) -> Any:
    eng = host.engine()
    target = eng.mcp_servers.get(server)
    if target is None:
        raise McpError(f"no MCP server named {server!r}")
    body = json.dumps(params if params is not None else {})
    if hasattr(target, "mcp_call"):                       # a client session: relay over its socket
        fut = asyncio.run_coroutine_threadsafe(target.mcp_call(host.proc().id, server, method, body), target.loop)
        ok, result = await asyncio.wrap_future(fut)
    else:                                                  # in-process callable(method, params_json) -> str
        try:
            r = target(method, body)
            if inspect.isawaitable(r):
                r = await r
            ok, result = True, r
        except Exception as e:  # noqa: BLE001
            ok, result = False, str(e)
    if not ok:
        raise McpError(str(result))
    try:
        return json.loads(result)
    except (TypeError, json.JSONDecodeError):
        return result


async def list_tools(server: str) -> List[dict]:
    r = await request(server, "tools/list")
    return r.get("tools", r) if isinstance(r, dict) else r


async def call_tool(server: str, name: str, arguments: dict) -> Any:
    return await request(server, "tools/call", {"name": name, "arguments": arguments})
