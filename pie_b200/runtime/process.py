"""Inferlet processes.

One launched program = one process: a UUID, an admission slot, an event stream
(`stdout | stderr | message | return | error`) relayed to the attached client or kept in a
4096-entry ring while detached, a mailbox for client signals and file transfers, and the set
of contexts it owns (destroyed when the process ends).

Native inferlets are Python coroutines `async def main(input: dict) -> str | None` written
against :mod:`pie_b200.sdk`, whose surface mirrors the WIT world `pie:inferlet/inferlet`;
the current process is found through a context variable, the way a wasm instance finds its
store. Counterpart of runtime/src/process.rs:35-76 (events), :184-219 (spawn), :430-529 (run),
runtime/src/instance.rs:63-68 (contexts die with the instance).
"""
from __future__ import annotations

import asyncio
import contextvars
import io
import json
import time
import traceback
import uuid
from collections import deque
from dataclasses import dataclass
from typing import Any, Callable, Deque, Dict, List, Optional

from .policy import FsPolicy, NetworkPolicy

EVENT_RING = 4096
current_process: "contextvars.ContextVar[Process]" = contextvars.ContextVar("pie_process")


@dataclass
class ProcessEvent:
    process_id: str
    event: str      # stdout | stderr | message | return | error
    value: str


class Process:
    def __init__(self, engine, program: str, entry: Callable, input_value: Any, username: str = "local",
                 capture_outputs: bool = True, token_budget: Optional[int] = None, parent: Optional[str] = None):
        self.engine, self.program, self.entry = engine, program, entry
        self.input = input_value
        self.id = str(uuid.uuid4())
        self.username, self.capture_outputs = username, capture_outputs
        self.token_budget = token_budget
        self.tokens_used = 0
        self.parent = parent
        self.events: Deque[ProcessEvent] = deque(maxlen=EVENT_RING)
        self.listeners: List[Callable[[ProcessEvent], None]] = []
        self.mailbox: "asyncio.Queue[str]" = None
        self.files: "asyncio.Queue[bytes]" = None
        self.task: Optional[asyncio.Task] = None
        self.done = asyncio.Event() if False else None
        self.result: Optional[str] = None
        self.error: Optional[str] = None
        self.finished = False
        self.t_start = time.time()
        self.t_end: Optional[float] = None
        self._done_waiters: List[Callable] = []
        self.scratch_dir: Optional[str] = None
        self.fs_policy: Optional[FsPolicy] = None
        self.network_policy: Optional[NetworkPolicy] = None

    def scratch(self) -> str:
        """This process's private directory (created on first use; removed when it ends)."""
        if self.scratch_dir is None:
            pol = self.fs_policy or FsPolicy("none")
            self.scratch_dir = pol.make_scratch(self.id)
            if self.scratch_dir is None:
                from .policy import PolicyError
                raise PolicyError("this process has no filesystem access")
        return self.scratch_dir

    # ------------------------------------------------------------------ events
    def emit(self, event: str, value: str) -> None:
        ev = ProcessEvent(self.id, event, value)
        if self.listeners:
            for cb in list(self.listeners):
                try:
                    cb(ev)
                except Exception:  # a broken listener must not kill the inferlet
                    pass
        else:
            self.events.append(ev)

    def attach(self, cb: Callable[[ProcessEvent], None]) -> None:
        """Start relaying events to `cb`, first replaying what was buffered while detached."""
        while self.events:
            cb(self.events.popleft())
        self.listeners.append(cb)

    def detach(self, cb) -> None:
        if cb in self.listeners:
            self.listeners.remove(cb)

    def print(self, *args, err: bool = False) -> None:
        buf = io.StringIO()
        print(*args, file=buf, end="")
        self.emit("stderr" if err else "stdout", buf.getvalue())

    # ------------------------------------------------------------------ lifecycle
    async def run(self) -> None:
        eng = self.engine
        self.mailbox, self.files = asyncio.Queue(), asyncio.Queue()
        token = current_process.set(self)
        try:
            async with eng.admission:
                await eng.admit_process(self)
                self.fs_policy = FsPolicy(eng.config.fs_policy, eng.config.scratch_root)
                self.network_policy = NetworkPolicy(list(eng.config.network_allow))
                if self.program in getattr(eng, "confined_programs", ()):
                    from .policy import Confinement, confine
                    with confine(Confinement(self.program, network=self.network_policy, process=self)):
                        result = await self.entry(self.input)
                else:
                    result = await self.entry(self.input)
            if result is not None and not isinstance(result, str):
                result = json.dumps(result)
            self.result = result if result is not None else ""
            self.emit("return", self.result)
        except asyncio.CancelledError:
            self.error = "terminated"
            self.emit("error", "terminated")
        except BaseException as e:  # noqa: BLE001
            self.error = f"{type(e).__name__}: {e}"
            eng.log.debug("inferlet %s failed:\n%s", self.program, traceback.format_exc())
            self.emit("error", self.error)
        finally:
            current_process.reset(token)
            FsPolicy.drop_scratch(self.scratch_dir)
            self.finished = True
            self.t_end = time.time()
            eng.release_process(self)
            for cb in self._done_waiters:
                cb(self)

    def terminate(self) -> None:
        if self.task is not None and not self.task.done():
            self.task.cancel()

    def on_done(self, cb: Callable) -> None:
        if self.finished:
            cb(self)
        else:
            self._done_waiters.append(cb)

    def charge_tokens(self, n: int) -> None:
        self.tokens_used += n

    def budget_exhausted(self) -> bool:
        return self.token_budget is not None and self.tokens_used >= self.token_budget

    def stats(self) -> dict:
        return {"id": self.id, "program": self.program, "username": self.username,
                "finished": self.finished, "tokens_used": self.tokens_used,
                "elapsed_s": (self.t_end or time.time()) - self.t_start}
