"""Front door: WebSocket sessions speaking msgpack maps tagged by `type`, request/response
matched by `corr_id`; same message set as the reference's client protocol
(client/rust/src/message.rs:9-180; session handling runtime/src/server.rs:333-600,
server/handler.rs:353-887).

Client -> server: auth_identify, auth_prove, auth_by_token, check_program, query, add_program
(256 KiB chunks), launch_process, launch_processes, run_processes, launch_daemon,
attach_process, terminate_process, signal_process, transfer_file, list_processes, ping,
register_mcp_server, mcp_response, submit_workflow, cancel_workflow, attach_workflow,
detach_workflow. Server -> client: response, process_event, file, mcp_request.

Programs are native inferlets: the uploaded blob is Python source defining `async def main`,
stored under the program directory with its manifest and registered with the engine.
"""
from __future__ import annotations

import asyncio
import base64
import hashlib
import json
import random
import threading
import tomllib
from pathlib import Path
from typing import Any, Dict, Optional

import msgpack
import websockets

from ..runtime.engine import Engine
from ..runtime.process import ProcessEvent
from ..runtime.program import Manifest, ProgramError, ProgramStore
from ..runtime.workflow import WorkflowExecutor
from .auth import Authenticator

CHUNK_SIZE_BYTES = 256 * 1024
QUERY_MODEL_STATUS = "model_status"


def load_program_source(engine: Engine, name: str, source: str, manifest: Optional[dict] = None) -> None:
    """Register a native inferlet from Python source (must define `async def main(input)`)."""
    from ..runtime.program import ProgramError, compile_program
    try:
        entry = compile_program(name, source)
    except ProgramError as e:
        raise ValueError(str(e)) from None
    engine.register_program(name, entry, manifest, confined=True)


class Session:
    def __init__(self, server: "PieServer", ws):
        self.server, self.ws, self.engine = server, ws, server.engine
        self.authed = not server.auth.enabled
        self.username = "anonymous" if self.authed else ""
        self.challenge: Optional[bytes] = None
        self.pending_user = ""
        self.uploads: Dict[str, dict] = {}
        self.attached: Dict[str, Any] = {}
        self.file_rx: Dict[str, dict] = {}
        self.loop = asyncio.get_running_loop()
        self.mcp_waiters: Dict[int, asyncio.Future] = {}
        self._mcp_id = 0

    # ---- plumbing
    async def send(self, msg: dict) -> None:
        await self.ws.send(msgpack.packb(msg, use_bin_type=True))

    def send_threadsafe(self, msg: dict) -> None:
        asyncio.run_coroutine_threadsafe(self.send(msg), self.loop)

    async def respond(self, corr_id, ok: bool, result: Any = "") -> None:
        await self.send({"type": "response", "corr_id": corr_id, "ok": ok,
                         "result": result if isinstance(result, str) else json.dumps(result)})

    def _relay(self, ev: ProcessEvent) -> None:
        self.send_threadsafe({"type": "process_event", "process_id": ev.process_id, "event": ev.event, "value": ev.value})

    # ---- dispatch
    async def run(self) -> None:
        try:
            async for raw in self.ws:
                try:
                    msg = msgpack.unpackb(raw, raw=False)
                    await self.handle(msg)
                except Exception as e:  # noqa: BLE001 - a bad message must not end the session
                    cid = msg.get("corr_id") if isinstance(locals().get("msg"), dict) else None
                    if cid is not None:
                        await self.respond(cid, False, f"{type(e).__name__}: {e}")
        finally:
            for pid, cb in self.attached.items():
                p = self.engine.processes.get(pid)
                if p is not None:
                    p.detach(cb)

    async def handle(self, m: dict) -> None:
        t, cid = m.get("type"), m.get("corr_id")
        if t == "auth_identify":
            self.pending_user = m["username"]
            self.challenge = self.server.auth.new_challenge()
            return await self.respond(cid, True, base64.b64encode(self.challenge).decode())
        if t == "auth_prove":
            ok = self.challenge is not None and self.server.auth.check_signature(self.pending_user, self.challenge,
                                                                                 m["signature"])
            self.challenge = None
            if ok:
                self.authed, self.username = True, self.pending_user
            return await self.respond(cid, ok, "authenticated" if ok else "signature rejected")
        if t == "auth_by_token":
            ok = self.server.auth.check_token(m["token"])
            if not ok:
                await asyncio.sleep(random.uniform(1.0, 3.0) * self.server.bad_token_delay_scale)
            else:
                self.authed, self.username = True, "internal"
            return await self.respond(cid, ok, "authenticated" if ok else "invalid token")
        if t == "ping":
            return await self.respond(cid, True, "pong")
        if not self.authed:
            if cid is not None:
                await self.respond(cid, False, "not authenticated")
            return
        h = getattr(self, "on_" + str(t), None)
        if h is None:
            if cid is not None:
                await self.respond(cid, False, f"unknown message type {t!r}")
            return
        await h(m, cid)

    # ---- programs
    async def on_check_program(self, m, cid):
        name = m["name"]
        known = name in self.engine.programs
        if known and m.get("wasm_hash"):
            known = self.server.program_hashes.get(name) == m["wasm_hash"]
        await self.respond(cid, True, "true" if known else "false")

    async def on_add_program(self, m, cid):
        if not self.server.allow_program_upload:
            return await self.respond(cid, False, "uploads disabled: set [server] allow_program_upload = true "
                                                  "(uploaded programs run unsandboxed in the engine process)")
        key = m["program_hash"]
        up = self.uploads.setdefault(key, {"chunks": {}, "manifest": m["manifest"]})
        up["chunks"][m["chunk_index"]] = bytes(m["chunk_data"])
        if len(up["chunks"]) < m["total_chunks"]:
            return await self.respond(cid, True, "chunk accepted")
        blob = b"".join(up["chunks"][i] for i in range(m["total_chunks"]))
        del self.uploads[key]
        if hashlib.sha256(blob).hexdigest() != key:
            return await self.respond(cid, False, "program hash mismatch")
        try:
            manifest = Manifest.parse(up["manifest"] or "")
        except ProgramError as e:
            return await self.respond(cid, False, str(e))
        name = manifest.name
        if name in self.engine.programs and not m.get("force_overwrite"):
            return await self.respond(cid, False, f"program {name} exists")
        try:
            self.server.store.install(blob.decode("utf-8"), manifest)
        except (ProgramError, SyntaxError) as e:
            return await self.respond(cid, False, f"install failed: {e}")
        self.server.program_hashes[name] = key
        await self.respond(cid, True, name)

    # ---- processes
    def _launch(self, inferlet, input_str, capture, budget):
        try:
            inp = json.loads(input_str) if input_str else None
        except json.JSONDecodeError:
            inp = input_str
        proc = self.engine.launch(inferlet, inp, username=self.username, capture_outputs=capture, token_budget=budget,
                                  listener=self._relay if capture else None)
        if capture:
            self.attached[proc.id] = self._relay
        return proc

    async def on_launch_process(self, m, cid):
        proc = self._launch(m["inferlet"], m.get("input", ""), m.get("capture_outputs", True), m.get("token_budget"))
        await self.respond(cid, True, proc.id)

    async def on_launch_processes(self, m, cid):
        budgets = m.get("token_budgets") or [None] * len(m["inputs"])
        ids = [self._launch(m["inferlet"], i, m.get("capture_outputs", True), b).id for i, b in zip(m["inputs"], budgets)]
        await self.respond(cid, True, ids)

    async def on_run_processes(self, m, cid):
        """Launch a batch and answer once with every result (no event relay)."""
        budgets = m.get("token_budgets") or [None] * len(m["inputs"])
        procs = [self._launch(m["inferlet"], i, False, b) for i, b in zip(m["inputs"], budgets)]
        done = asyncio.Event()
        left = [len(procs)]

        def one(_p):
            left[0] -= 1
            if left[0] == 0:
                self.loop.call_soon_threadsafe(done.set)
        for p in procs:
            p.on_done(one)
        await done.wait()
        await self.respond(cid, True, [{"ok": p.error is None, "value": p.result if p.error is None else p.error}
                                       for p in procs])

    async def on_attach_process(self, m, cid):
        p = self.engine.processes.get(m["process_id"])
        if p is None:
            return await self.respond(cid, False, "no such process")
        self.attached[p.id] = self._relay
        p.attach(self._relay)
        await self.respond(cid, True, "attached")

    async def on_terminate_process(self, m, cid):
        await self.respond(cid, self.engine.terminate(m["process_id"]), "")

    async def on_signal_process(self, m, cid):
        p = self.engine.processes.get(m["process_id"])
        if p is not None and p.mailbox is not None:
            self.engine.call_soon(p.mailbox.put_nowait, m["message"])

    async def on_transfer_file(self, m, cid):
        st = self.file_rx.setdefault(m["file_hash"], {})
        st[m["chunk_index"]] = bytes(m["chunk_data"])
        if len(st) == m["total_chunks"]:
            blob = b"".join(st[i] for i in range(m["total_chunks"]))
            del self.file_rx[m["file_hash"]]
            p = self.engine.processes.get(m["process_id"])
            if p is not None and p.files is not None:
                self.engine.call_soon(p.files.put_nowait, blob)

    async def on_list_processes(self, m, cid):
        await self.respond(cid, True, self.engine.list_processes())

    async def on_query(self, m, cid):
        if m["subject"] == QUERY_MODEL_STATUS:
            return await self.respond(cid, True, self.engine.model_status())
        if m["subject"] == "programs":
            return await self.respond(cid, True, sorted(self.engine.programs))
        if m["subject"] == "version":
            from ..runtime.engine import VERSION
            return await self.respond(cid, True, VERSION)
        await self.respond(cid, False, f"unknown query subject {m['subject']!r}")

    async def on_launch_daemon(self, m, cid):
        from .daemon import start_daemon
        port = await start_daemon(self.engine, m["inferlet"], m.get("input", ""), int(m["port"]), self.username)
        await self.respond(cid, True, str(port))

    # ---- MCP relay: inferlets call tools hosted by the client
    async def on_register_mcp_server(self, m, cid):
        self.engine.mcp_servers[m["name"]] = self
        await self.respond(cid, True, m["name"])

    async def on_mcp_response(self, m, cid):
        fut = self.mcp_waiters.pop(cid, None)
        if fut is not None and not fut.done():
            fut.set_result((m["ok"], m["result"]))

    async def mcp_call(self, process_id: str, server_name: str, method: str, params: str):
        self._mcp_id += 1
        cid = 1_000_000 + self._mcp_id
        fut = self.loop.create_future()
        self.mcp_waiters[cid] = fut
        await self.send({"type": "mcp_request", "corr_id": cid, "process_id": process_id, "server_name": server_name,
                         "method": method, "params": params})
        return await asyncio.wait_for(fut, 60)

    # ---- workflows
    async def on_submit_workflow(self, m, cid):
        wid = self.server.workflows.submit(json.loads(m["json"]), self.username, listener=self._wf_event)
        await self.respond(cid, True, wid)

    def _wf_event(self, wid, event, value):
        self.send_threadsafe({"type": "process_event", "process_id": wid, "event": event, "value": value})

    async def on_cancel_workflow(self, m, cid):
        await self.respond(cid, self.server.workflows.cancel(m["workflow_id"]), "")

    async def on_attach_workflow(self, m, cid):
        await self.respond(cid, self.server.workflows.attach(m["workflow_id"], self._wf_event), "")

    async def on_detach_workflow(self, m, cid):
        await self.respond(cid, self.server.workflows.detach(m["workflow_id"], self._wf_event), "")


class PieServer:
    def __init__(self, engine: Engine, host: str = "127.0.0.1", port: int = 8080, auth: Optional[Authenticator] = None,
                 program_dir: Optional[str] = None, max_message_bytes: int = 64 << 20, registry_url: str = "",
                 allow_program_upload: bool = False):
        self.engine, self.host, self.port = engine, host, port
        # Programs are native Python and run in this process with its privileges; uploads (and the
        # programs an earlier run cached on disk) are only accepted when the operator opted in.
        self.allow_program_upload = allow_program_upload
        self.auth = auth or Authenticator(False)
        self.program_dir = Path(program_dir).expanduser() if program_dir else None
        self.program_hashes: Dict[str, str] = {}
        self.workflows = WorkflowExecutor(engine)
        self.max_message_bytes = max_message_bytes
        self.bad_token_delay_scale = 1.0
        self.loop: Optional[asyncio.AbstractEventLoop] = None
        self._server = None
        self._thread: Optional[threading.Thread] = None
        self._ready = threading.Event()
        self.store = ProgramStore(engine, str(self.program_dir) if self.program_dir else None, registry_url)
        if registry_url:
            engine.program_resolver = self.store.ensure
        self._load_stored_programs()

    def _load_stored_programs(self) -> None:
        """Programs installed earlier (disk cache programs/<name>/<version>.{py,toml})."""
        if not self.allow_program_upload:
            return
        try:
            for ref in self.store.load_cache():
                name, _, ver = ref.partition("@")
                src = self.program_dir / name / f"{ver}.py"
                self.program_hashes[name] = hashlib.sha256(src.read_bytes()).hexdigest()
        except Exception:  # noqa: BLE001 - a broken cached program must not stop the server
            pass

    async def _handler(self, ws):
        await Session(self, ws).run()

    async def _main(self):
        self._server = await websockets.serve(self._handler, self.host, self.port, max_size=self.max_message_bytes)
        self.port = self._server.sockets[0].getsockname()[1]
        self._ready.set()
        await self._server.wait_closed()

    def start(self) -> int:
        """Serve on a background thread; returns the bound port (port 0 = pick a free one)."""
        def run():
            self.loop = asyncio.new_event_loop()
            asyncio.set_event_loop(self.loop)
            self.loop.run_until_complete(self._main())
        self._thread = threading.Thread(target=run, name="pie-server", daemon=True)
        self._thread.start()
        self._ready.wait(10)
        return self.port

    def stop(self) -> None:
        if self._server is not None and self.loop is not None:
            self.loop.call_soon_threadsafe(self._server.close)
        if self._thread is not None:
            self._thread.join(timeout=5)
