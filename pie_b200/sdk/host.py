"""Bridge between SDK objects and the engine for the calling inferlet process.

The functions here are the native form of the WIT host imports (`pie:core/*`): each takes the
current process from a context variable (the wasm instance's store in the reference,
runtime/src/api.rs:43-129) and calls into the engine's services.
"""
from __future__ import annotations

import asyncio

from ..runtime.inference import Future
from ..runtime.process import Process, current_process


def proc() -> Process:
    try:
        return current_process.get()
    except LookupError:
        raise RuntimeError("SDK call outside of an inferlet process") from None


def engine():
    return proc().engine


class _Mailbox:
    """Completions from runtime threads to one event loop, delivered in batches: a completion is pushed
    on a deque and the loop is woken (one write to its self-pipe) only when no drain is pending, so a
    batch of several hundred futures finished by one fire costs one wake-up instead of one each."""

    def __init__(self, loop):
        import collections
        import threading
        self.loop = loop
        self.items = collections.deque()
        self.lock = threading.Lock()
        self.scheduled = False

    def post(self, afut, f: Future) -> None:
        with self.lock:
            self.items.append((afut, f))
            if self.scheduled:
                return
            self.scheduled = True
        self.loop.call_soon_threadsafe(self.drain)

    def drain(self) -> None:
        while True:
            with self.lock:
                if not self.items:
                    self.scheduled = False
                    return
                batch = list(self.items)
                self.items.clear()
            for afut, f in batch:
                _resolve(afut, f)


def _mailbox(loop) -> _Mailbox:
    mb = getattr(loop, "_pie_mailbox", None)
    if mb is None:
        mb = loop._pie_mailbox = _Mailbox(loop)
    return mb


async def wait(fut: Future):
    """Await a runtime future from the inferlet's coroutine."""
    if fut.done():
        return fut.result()
    loop = asyncio.get_running_loop()
    afut = loop.create_future()
    mb = _mailbox(loop)
    fut.add_done_callback(lambda f: mb.post(afut, f))
    return await afut


def _resolve(afut, f: Future):
    if afut.done():
        return
    try:
        afut.set_result(f.result())
    except BaseException as e:  # noqa: BLE001
        afut.set_exception(e)
