"""Python client of the engine's WebSocket + msgpack protocol (synchronous facade over a
background asyncio loop). Mirrors the reference client (client/python/src/pie_client/client.py,
client/rust/src/client.rs): authenticate by token or key, install programs in 256 KiB chunks,
launch / attach / signal / terminate processes, stream their events, query status, submit
workflows, and host MCP tools for inferlets."""
from __future__ import annotations

import asyncio
import base64
import hashlib
import json
import queue
import threading
from typing import Any, Callable, Dict, List, Optional

import msgpack
import websockets

CHUNK = 256 * 1024


class ClientError(RuntimeError):
    pass


class ProcessHandle:
    def __init__(self, client: "PieClient", pid: str):
        self.client, self.id = client, pid
        self.events: "queue.Queue[tuple]" = queue.Queue()
        self.files: "queue.Queue[bytes]" = queue.Queue()

    def recv(self, timeout: Optional[float] = None) -> tuple:
        """Next (event, value): stdout | stderr | message | return | error."""
        return self.events.get(timeout=timeout)

    def wait(self, timeout: float = 600.0) -> str:
        """Drain events until the process returns; raises on an error event."""
        while True:
            ev, val = self.recv(timeout)
            if ev == "return":
                return val
            if ev == "error":
                raise ClientError(val)

    def signal(self, message: str) -> None:
        self.client._send({"type": "signal_process", "process_id": self.id, "message": message})

    def transfer_file(self, data: bytes) -> None:
        h = hashlib.sha256(data).hexdigest()
        n = max(1, -(-len(data) // CHUNK))
        for i in range(n):
            self.client._send({"type": "transfer_file", "process_id": self.id, "file_hash": h, "chunk_index": i,
                               "total_chunks": n, "chunk_data": data[i * CHUNK:(i + 1) * CHUNK]})

    def terminate(self) -> bool:
        return self.client._request({"type": "terminate_process", "process_id": self.id})[0]


class PieClient:
    def __init__(self, uri: str, timeout: float = 30.0):
        self.uri, self.timeout = uri, timeout
        self.loop = asyncio.new_event_loop()
        self._corr = 0
        self._waiters: Dict[int, "queue.Queue"] = {}
        self._procs: Dict[str, ProcessHandle] = {}
        self._orphans: Dict[str, list] = {}
        self._file_rx: Dict[str, dict] = {}
        self.mcp_tools: Dict[str, Callable[[str, str], str]] = {}
        self._ws = None
        self._ready = threading.Event()
        self._err: Optional[BaseException] = None
        self._thread = threading.Thread(target=self._run, name="pie-client", daemon=True)
        self._thread.start()
        if not self._ready.wait(timeout) or self._err:
            raise ClientError(f"cannot connect to {uri}: {self._err}")

    # ---- transport
    def _run(self):
        asyncio.set_event_loop(self.loop)
        try:
            self.loop.run_until_complete(self._main())
        except BaseException as e:  # noqa: BLE001
            self._err = e
            self._ready.set()

    async def _main(self):
        async with websockets.connect(self.uri, max_size=64 << 20) as ws:
            self._ws = ws
            self._ready.set()
            async for raw in ws:
                self._on_message(msgpack.unpackb(raw, raw=False))

    def _on_message(self, m: dict) -> None:
        t = m.get("type")
        if t == "response":
            w = self._waiters.pop(m["corr_id"], None)
            if w is not None:
                w.put((m["ok"], m["result"]))
        elif t == "process_event":
            h = self._procs.get(m["process_id"])
            if h is not None:
                h.events.put((m["event"], m["value"]))
            else:
                self._orphans.setdefault(m["process_id"], []).append((m["event"], m["value"]))
        elif t == "file":
            st = self._file_rx.setdefault(m["file_hash"], {})
            st[m["chunk_index"]] = bytes(m["chunk_data"])
            if len(st) == m["total_chunks"]:
                blob = b"".join(st[i] for i in range(m["total_chunks"]))
                del self._file_rx[m["file_hash"]]
                h = self._procs.get(m["process_id"])
                if h is not None:
                    h.files.put(blob)
        elif t == "mcp_request":
            fn = self.mcp_tools.get(m["server_name"])
            try:
                ok, res = (True, fn(m["method"], m["params"])) if fn else (False, "no such MCP server")
            except Exception as e:  # noqa: BLE001
                ok, res = False, str(e)
            asyncio.ensure_future(self._ws.send(msgpack.packb(
                {"type": "mcp_response", "corr_id": m["corr_id"], "ok": ok, "result": res}, use_bin_type=True)))

    def _send(self, msg: dict) -> None:
        asyncio.run_coroutine_threadsafe(self._ws.send(msgpack.packb(msg, use_bin_type=True)), self.loop).result(self.timeout)

    def _request(self, msg: dict, timeout: Optional[float] = None):
        self._corr += 1
        cid = self._corr
        q: "queue.Queue" = queue.Queue()
        self._waiters[cid] = q
        self._send(dict(msg, corr_id=cid))
        try:
            return q.get(timeout=timeout or self.timeout)
        except queue.Empty:
            raise ClientError(f"no response to {msg.get('type')}") from None

    def _ok(self, msg: dict, timeout: Optional[float] = None) -> str:
        ok, res = self._request(msg, timeout)
        if not ok:
            raise ClientError(res)
        return res

    # ---- API
    def ping(self) -> str:
        return self._ok({"type": "ping"})

    def auth_by_token(self, token: str) -> None:
        self._ok({"type": "auth_by_token", "token": token})

    def auth_with_key(self, username: str, private_key) -> None:
        from ..server.auth import sign
        challenge = base64.b64decode(self._ok({"type": "auth_identify", "username": username}))
        self._ok({"type": "auth_prove", "signature": base64.b64encode(sign(private_key, challenge)).decode()})

    def query(self, subject: str, record: str = "") -> Any:
        res = self._ok({"type": "query", "subject": subject, "record": record})
        try:
            return json.loads(res)
        except json.JSONDecodeError:
            return res

    def model_status(self) -> dict:
        return self.query("model_status")

    def program_exists(self, name: str, version: str = "", program_hash: Optional[str] = None) -> bool:
        return self._ok({"type": "check_program", "name": name, "version": version, "wasm_hash": program_hash}) == "true"

    def install_program(self, source: bytes, manifest: str, force: bool = True) -> str:
        h = hashlib.sha256(source).hexdigest()
        n = max(1, -(-len(source) // CHUNK))
        res = ""
        for i in range(n):
            res = self._ok({"type": "add_program", "program_hash": h, "manifest": manifest, "force_overwrite": force,
                            "chunk_index": i, "total_chunks": n, "chunk_data": source[i * CHUNK:(i + 1) * CHUNK]})
        return res

    def launch_process(self, inferlet: str, input_value: Any = None, capture_outputs: bool = True,
                       token_budget: Optional[int] = None) -> ProcessHandle:
        inp = input_value if isinstance(input_value, str) else json.dumps(input_value)
        pid = self._ok({"type": "launch_process", "inferlet": inferlet, "input": inp, "capture_outputs": capture_outputs,
                        "token_budget": token_budget})
        h = ProcessHandle(self, pid)
        self._procs[pid] = h
        for ev in self._orphans.pop(pid, []):
            h.events.put(ev)
        return h

    def run_processes(self, inferlet: str, inputs: List[Any], timeout: float = 600.0) -> List[dict]:
        ins = [i if isinstance(i, str) else json.dumps(i) for i in inputs]
        return json.loads(self._ok({"type": "run_processes", "inferlet": inferlet, "inputs": ins}, timeout))

    def attach_process(self, pid: str) -> ProcessHandle:
        h = self._procs.setdefault(pid, ProcessHandle(self, pid))
        self._ok({"type": "attach_process", "process_id": pid})
        return h

    def list_processes(self) -> List[dict]:
        return json.loads(self._ok({"type": "list_processes"}))

    def launch_daemon(self, inferlet: str, port: int, input_value: Any = None) -> int:
        inp = input_value if isinstance(input_value, str) else json.dumps(input_value or {})
        return int(self._ok({"type": "launch_daemon", "port": port, "inferlet": inferlet, "input": inp}))

    def register_mcp_server(self, name: str, fn: Callable[[str, str], str]) -> None:
        self.mcp_tools[name] = fn
        self._ok({"type": "register_mcp_server", "name": name, "transport": "client"})

    def submit_workflow(self, spec: dict) -> ProcessHandle:
        wid = self._ok({"type": "submit_workflow", "json": json.dumps(spec)})
        h = ProcessHandle(self, wid)
        self._procs[wid] = h
        for ev in self._orphans.pop(wid, []):
            h.events.put(ev)
        return h

    def cancel_workflow(self, wid: str) -> bool:
        return self._request({"type": "cancel_workflow", "workflow_id": wid})[0]

    def close(self) -> None:
        if self._ws is not None:
            try:
                asyncio.run_coroutine_threadsafe(self._ws.close(), self.loop).result(5)
            except Exception:  # noqa: BLE001
                pass
        self._thread.join(timeout=5)
