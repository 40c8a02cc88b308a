"""WIT `runtime` interface: version, instance id, username, models, launch child processes.
Counterpart of runtime/src/api/runtime.rs:53-92 (launch returns a pollable child)."""
from __future__ import annotations

import asyncio
from typing import Any, List, Optional

from . import host


def version() -> str:
    from ..runtime.engine import VERSION
    return VERSION


def instance_id() -> str:
    return host.proc().id


def username() -> str:
    return host.proc().username


def models() -> List[str]:
    return list(host.engine().models)


def args() -> Any:
    return host.proc().input


def print_out(*a) -> None:
    host.proc().print(*a)


def print_err(*a) -> None:
    host.proc().print(*a, err=True)


class Child:
    def __init__(self, proc):
        self._proc = proc
        self._ev = asyncio.Event()
        loop = asyncio.get_running_loop()
        proc.on_done(lambda _p: loop.call_soon_threadsafe(self._ev.set))

    def pid(self) -> str:
        return self._proc.id

    def get(self) -> Optional[str]:
        if not self._proc.finished:
            return None
        if self._proc.error is not None:
            raise RuntimeError(self._proc.error)
        return self._proc.result

    async def wait(self) -> str:
        await self._ev.wait()
        return self.get()

    def cancel(self) -> None:
        self._proc.terminate()


def launch(program: str, input_value: Any = None) -> Child:
    p = host.proc()
    child = p.engine.launch(program, input_value, username=p.username, capture_outputs=False, parent=p.id)
    return Child(child)
