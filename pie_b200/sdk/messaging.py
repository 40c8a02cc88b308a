"""WIT `messaging` interface: push / pull queues and broadcast / subscribe topics."""
from __future__ import annotations

from . import host


def push(topic: str, message: str) -> None:
    host.engine().messaging.push(topic, message)


async def pull(topic: str) -> str:
    return await host.engine().messaging.pull(topic)


def broadcast(topic: str, message: str) -> None:
    host.engine().messaging.broadcast(topic, message)


def subscribe(topic: str):
    return host.engine().messaging.subscribe(topic)
