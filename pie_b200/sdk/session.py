"""WIT `session` interface: messages and files between the inferlet and its client."""
from __future__ import annotations

from . import host


def send(message: str) -> None:
    host.proc().emit("message", message)


async def receive() -> str:
    return await host.proc().mailbox.get()


def send_file(data: bytes) -> None:
    p = host.proc()
    p.engine.deliver_file(p, data) if hasattr(p.engine, "deliver_file") else p.emit("message", f"<file {len(data)} bytes>")


async def receive_file() -> bytes:
    return await host.proc().files.get()
