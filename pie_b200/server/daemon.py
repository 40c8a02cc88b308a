"""Daemons: a long-lived inferlet bound to a TCP port; every HTTP request launches the program with
{"method", "path", "headers", "body", plus the daemon's static input} and its return value is the
response body (JSON return `{"status", "headers", "body"}` sets those explicitly). `GET /metrics`
is answered by the engine itself with its Prometheus exposition.
Counterpart of runtime/src/daemon.rs:1-90 (wasi:http incoming-handler served with hyper)."""
from __future__ import annotations

import asyncio
import json
from typing import Dict

_DAEMONS: Dict[int, asyncio.AbstractServer] = {}


async def start_daemon(engine, program: str, static_input: str, port: int, username: str = "local") -> int:
    try:
        static = json.loads(static_input) if static_input else {}
    except json.JSONDecodeError:
        static = {"input": static_input}

    async def handle(reader: asyncio.StreamReader, writer: asyncio.StreamWriter):
        try:
            head = await reader.readuntil(b"\r\n\r\n")
            lines = head.decode("latin1").split("\r\n")
            method, path, _ = lines[0].split(" ", 2)
            headers = {k.strip().lower(): v.strip() for k, v in (l.split(":", 1) for l in lines[1:] if ":" in l)}
            n = int(headers.get("content-length", "0"))
            body = (await reader.readexactly(n)).decode("utf-8", errors="replace") if n else ""
            if method == "GET" and path == "/metrics":
                data = engine.metrics_text().encode("utf-8")
                writer.write(b"HTTP/1.1 200 OK\r\ncontent-type: text/plain; version=0.0.4\r\ncontent-length: "
                             + str(len(data)).encode() + b"\r\nconnection: close\r\n\r\n" + data)
                await writer.drain()
                return
            req = dict(static, method=method, path=path, headers=headers, body=body)
            proc = engine.launch(program, req, username=username, capture_outputs=False)
            ev = asyncio.Event()
            loop = asyncio.get_running_loop()
            proc.on_done(lambda _p: loop.call_soon_threadsafe(ev.set))
            await ev.wait()
            status, hdrs, out = (200, {}, proc.result or "") if proc.error is None else (500, {}, proc.error)
            try:
                j = json.loads(out)
                if isinstance(j, dict) and "body" in j and ("status" in j or "headers" in j):
                    status, hdrs, out = int(j.get("status", 200)), j.get("headers", {}), str(j["body"])
            except (json.JSONDecodeError, TypeError):
                pass
            data = out.encode("utf-8")
            hdrs = {"content-type": "text/plain; charset=utf-8", **hdrs, "content-length": str(len(data)),
                    "connection": "close"}
            writer.write(f"HTTP/1.1 {status} OK\r\n".encode() + "".join(f"{k}: {v}\r\n" for k, v in hdrs.items()).encode()
                         + b"\r\n" + data)
            await writer.drain()
        except Exception:  # noqa: BLE001 - a malformed request only closes its connection
            pass
        finally:
            writer.close()

    srv = await asyncio.start_server(handle, "127.0.0.1", port)
    bound = srv.sockets[0].getsockname()[1]
    _DAEMONS[bound] = srv
    return bound


async def stop_daemon(port: int) -> bool:
    srv = _DAEMONS.pop(port, None)
    if srv is None:
        return False
    srv.close()
    await srv.wait_closed()
    return True
