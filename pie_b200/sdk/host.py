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


async def wait(fut: Future):
    """Await a runtime future from the inferlet's coroutine."""
    if fut.done():
        return fut.result()
    loop = asyncio.get_running_loop()
    afut = loop.create_future()

    def done(f: Future):
        loop.call_soon_threadsafe(_resolve, afut, f)

    fut.add_done_callback(done)
    return await afut


def _resolve(afut, f: Future):
    if afut.done():
        return
    try:
        afut.set_result(f.result())
    except BaseException as e:  # noqa: BLE001
        afut.set_exception(e)
