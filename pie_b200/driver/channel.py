"""Channels between the runtime and a driver, and the driver proxy that speaks them.

A channel carries operations (`FORWARD`, `DECODE`, `COPY`, `CONTROL`) to the thread or process that owns the
driver and brings the answers back through tickets:

* `InProcChannel` - blocking: a heap queue and a condition variable; the driver thread gets the request
  object itself, nothing is serialised (runtime/src/driver/inproc.rs:1-140).
* `PollingChannel` - a fixed ring of generation-tagged slots that the driver thread polls with a spin
  budget before it parks; the `latency` profile (runtime/src/driver/inproc_polling.rs:1-120).
* `ShmemChannel` - another process: wire frames (`driver/abi.py`) through the native shared-memory slot
  ring (`csrc/host/shm_channel.hpp`), token-only answers on the 20-byte fast path
  (runtime/src/driver/shmem.rs:20-154, driver/bridge/src/ipc.rs).

`ChannelDriver` is a driver whose methods go through a channel, so the engine can sit on any of the
three without knowing (`runtime/src/driver.rs:36-158`: submit / submit_sync / notify / abort).
`serve(driver, channel)` is the loop on the driver's side; `python -m pie_b200.driver.channel --serve NAME`
runs it in a process of its own (service/inproc_service.cpp:31-191 is the reference's method switch).
"""
from __future__ import annotations

import heapq
import base64
import itertools
import os
import threading
import time
from dataclasses import asdict
from typing import Any, Callable, List, Optional

import numpy as np

from . import abi
from .schema import Capabilities, CopyRequest, ForwardRequest, ForwardResponse, SlotOutput

OP_FORWARD, OP_DECODE, OP_COPY, OP_CONTROL = 1, 2, 3, 4


class ChannelClosed(RuntimeError):
    pass


class ChannelTimeout(TimeoutError):
    pass


class Ticket:
    """The pending answer of one submitted operation."""
    __slots__ = ("_ev", "_value", "_error", "aborted", "t_submit")

    def __init__(self):
        self._ev = threading.Event()
        self._value, self._error, self.aborted = None, None, False
        self.t_submit = time.perf_counter()

    def set(self, value=None, error: Optional[BaseException] = None) -> None:
        self._value, self._error = value, error
        self._ev.set()

    def done(self) -> bool:
        return self._ev.is_set()

    def result(self, timeout: Optional[float] = None):
        if not self._ev.wait(timeout):
            self.aborted = True                    # the server drops the answer of an abandoned ticket
            raise ChannelTimeout("driver did not answer in time")
        if self._error is not None:
            raise self._error
        return self._value


def dispatch(driver, op: int, payload):
    """The driver-side method switch."""
    if op == OP_FORWARD:
        return driver.fire_batch(payload)
    if op == OP_DECODE:
        step, parity = payload
        return driver.decode_async(step, parity).wait()
    if op == OP_COPY:
        return driver.copy(payload)
    if op == OP_CONTROL:
        name = payload["op"]
        if name == "caps":
            return asdict(driver.capabilities())
        if name == "health":
            return bool(driver.health()) if hasattr(driver, "health") else True
        if name == "shutdown":
            if hasattr(driver, "shutdown"):
                driver.shutdown()
            return True
        if name in ("create_adapter", "destroy_adapter", "fork_adapter", "save_adapter", "load_adapter", "zo_apply",
                    "copy_rs", "release_media"):
            return getattr(driver, name)(*payload.get("args", []))
        if name == "put_media":
            # patch rows cross the control plane as base64 float16 (a cold path: once per image)
            slot, kind, b64, shape, grids = payload["args"]
            patches = np.frombuffer(base64.b64decode(b64), dtype=np.float16).reshape(shape).astype(np.float32)
            return driver.put_media(slot, kind, patches, grids)
        raise ValueError(f"unknown control operation {name!r}")
    raise ValueError(f"unknown operation {op}")


# ----------------------------------------------------------------------------- in-process, blocking
class InProcChannel:
    """Heap queue (priority, then arrival) + condition variable; one service thread owns the driver."""

    def __init__(self, driver, name: str = "pie-driver"):
        self.driver = driver
        self._heap: List[tuple] = []
        self._seq = itertools.count()
        self._cv = threading.Condition()
        self._closed: Optional[BaseException] = None
        self.served = 0
        self.thread = threading.Thread(target=self._serve, name=name, daemon=True)
        self.thread.start()

    def submit(self, op: int, payload, priority: int = 0) -> Ticket:
        t = Ticket()
        with self._cv:
            if self._closed is not None:
                raise ChannelClosed(str(self._closed))
            heapq.heappush(self._heap, (priority, next(self._seq), op, payload, t))
            self._cv.notify()
        return t

    def submit_sync(self, op: int, payload, timeout: Optional[float] = None):
        return self.submit(op, payload).result(timeout)

    def notify(self) -> None:
        with self._cv:
            self._cv.notify_all()

    def abort(self, reason: str = "aborted") -> None:
        """Fail everything queued and refuse new work; the operation being served finishes."""
        err = ChannelClosed(reason)
        with self._cv:
            self._closed = err
            pending, self._heap = self._heap, []
            self._cv.notify_all()
        for _, _, _, _, t in pending:
            t.set(error=err)

    def close(self) -> None:
        self.abort("channel closed")
        self.thread.join(timeout=5.0)

    def _serve(self) -> None:
        while True:
            with self._cv:
                while not self._heap and self._closed is None:
                    self._cv.wait()
                if self._closed is not None:
                    return
                _, _, op, payload, t = heapq.heappop(self._heap)
            if t.aborted:
                continue
            try:
                t.set(dispatch(self.driver, op, payload))
            except BaseException as e:  # noqa: BLE001 - the error belongs to the caller
                t.set(error=e)
            self.served += 1


# ----------------------------------------------------------------------------- in-process, polling
class PollingChannel:
    """The `latency` profile: a fixed ring of generation-tagged slots (native `PollRing`). The driver
    thread polls the head slot without the interpreter lock, spinning `spin_budget` rounds before it
    parks (a negative budget spins for ever: lowest latency, one busy core); a caller waits for its own
    slot the same way. Requests and answers stay Python objects, indexed by slot."""

    class _Pending:
        __slots__ = ("ch", "seq", "_value", "_taken")

        def __init__(self, ch, seq):
            self.ch, self.seq, self._taken = ch, seq, False

        def done(self) -> bool:
            return self._taken or self.ch.ring.is_done(self.seq)

        def result(self, timeout: Optional[float] = None):
            if not self._taken:
                c = self.ch
                if not c.ring.wait_done(self.seq, 3600.0 if timeout is None else timeout):
                    if c._closed is not None:
                        raise c._closed
                    c._abandoned.add(self.seq)              # the server releases the slot when it gets there
                    raise ChannelTimeout("driver did not answer in time")
                i = self.seq % c.n
                self._value, c.results[i] = c.results[i], None
                c.ring.release(self.seq)
                self._taken = True
            ok, val = self._value
            if not ok:
                raise val
            return val

    def __init__(self, driver, slots: int = 1024, spin_budget: int = 20000, name: str = "pie-driver-poll"):
        from .._C import pie_host
        self.driver, self.n = driver, slots
        self.ring = pie_host.PollRing(slots, spin_budget)
        self.items: List[Any] = [None] * slots
        self.results: List[Any] = [None] * slots
        self._abandoned: set = set()
        self._closed: Optional[BaseException] = None
        self.served = 0
        self.thread = threading.Thread(target=self._serve, name=name, daemon=True)
        self.thread.start()

    @property
    def parks(self) -> int:
        return self.ring.parks

    def submit(self, op: int, payload, priority: int = 0):
        seq = self.ring.claim()
        if seq == -2 or self._closed is not None:
            raise ChannelClosed(str(self._closed or "channel closed"))
        if seq < 0:
            raise ChannelClosed("driver ring is full")                # a whole lap in flight: the driver is gone
        self.items[seq % self.n] = (op, payload)
        self.ring.publish(seq)
        return PollingChannel._Pending(self, seq)

    def submit_sync(self, op: int, payload, timeout: Optional[float] = None):
        return self.submit(op, payload).result(timeout)

    def notify(self) -> None:
        pass                                                            # publish wakes a parked poller

    def abort(self, reason: str = "aborted") -> None:
        """Fail what is queued and refuse new work; the operation being served finishes."""
        self._closed = ChannelClosed(reason)
        self.ring.close()

    def close(self) -> None:
        self.abort("channel closed")
        self.thread.join(timeout=5.0)

    def _serve(self) -> None:
        ring = self.ring
        while True:
            seq = ring.poll(0.25)
            if seq == -2:
                break
            if seq < 0:
                continue
            i = seq % self.n
            op, payload = self.items[i]
            self.items[i] = None
            try:
                self.results[i] = (True, dispatch(self.driver, op, payload))
            except BaseException as e:  # noqa: BLE001
                self.results[i] = (False, e)
            self.served += 1
            if seq in self._abandoned:
                self._abandoned.discard(seq)
                self.results[i] = None
                ring.release(seq)
            else:
                ring.complete(seq)
        # closed: fail the requests that were published and never served
        err = self._closed or ChannelClosed("channel closed")
        for seq in range(ring.head, ring.tail):
            i = seq % self.n
            if self.items[i] is not None:
                self.items[i] = None
                self.results[i] = (False, err)
                ring.complete(seq)


# ----------------------------------------------------------------------------- another process
def _schema_hash64() -> int:
    return int(abi.schema_hash()[:16], 16)


class ShmemChannel:
    """Client end of the shared-memory slot ring: operations leave as wire frames, answers come back as
    frames (or as the token fast path) and are decoded on the caller's thread."""

    def __init__(self, name: str, create: bool = True, slots: int = 64, req_capacity: int = 8 << 20,
                 resp_capacity: int = 8 << 20, timeout_s: float = 120.0, spin_iters: int = 2000):
        from .._C import pie_host
        self.name, self.timeout_s = name, timeout_s
        self.ring = pie_host.ShmChannel(name, create, slots, req_capacity, resp_capacity, abi.SCHEMA_VERSION,
                                        _schema_hash64(), spin_iters)
        self.last_queue_us = self.last_service_us = 0.0

    @staticmethod
    def _encode(op: int, payload) -> bytes:
        if op == OP_FORWARD:
            return abi.pack_forward_request(payload)
        if op == OP_DECODE:
            return abi.pack_decode_step(*payload)
        if op == OP_COPY:
            return abi.pack_copy_request(payload)
        return abi.pack_control(payload)

    @staticmethod
    def _decode(op: int, buf: bytes):
        if abi.is_token_frame(buf):
            toks, fwd, tot = abi.unpack_tokens(buf)
            if op == OP_DECODE:
                return toks
            return ForwardResponse([SlotOutput("token", token=int(t)) for t in toks], toks, t_forward_us=fwd, t_total_us=tot)
        kind = abi.frame_kind(buf)
        if kind == abi.KIND_FORWARD_RESPONSE:
            return abi.unpack_forward_response(buf)
        res = abi.unpack_control(buf)
        if "error" in res:
            raise RuntimeError(f"driver: {res['error']}")
        return res.get("value")

    class _Pending:
        def __init__(self, ch, op, slot):
            self.ch, self.op, self.slot = ch, op, slot

        def done(self) -> bool:
            return self.ch.ring.slot_state(self.slot) == 4

        def result(self, timeout: Optional[float] = None):
            got = self.ch.ring.wait_response(self.slot, self.ch.timeout_s if timeout is None else timeout)
            if got is None:
                raise ChannelTimeout("driver process did not answer in time")
            buf, self.ch.last_queue_us, self.ch.last_service_us = got
            return ShmemChannel._decode(self.op, buf)

    def submit(self, op: int, payload, priority: int = 0):
        frame = self._encode(op, payload)
        deadline = time.monotonic() + self.timeout_s
        while True:
            slot = self.ring.submit(frame)
            if slot >= 0:
                return ShmemChannel._Pending(self, op, slot)
            if slot == -2:
                raise ChannelClosed("driver channel closed")
            if time.monotonic() > deadline:
                raise ChannelTimeout("no free slot in the driver channel")
            time.sleep(0.0005)

    def submit_sync(self, op: int, payload, timeout: Optional[float] = None):
        return self.submit(op, payload).result(timeout)

    def notify(self) -> None:
        pass                                    # every submit wakes a parked server

    def abort(self, reason: str = "aborted") -> None:
        self.ring.close()

    def close(self) -> None:
        self.ring.close()


def serve_shm(driver, name: str, idle_timeout_s: float = 0.5, stop: Optional[Callable[[], bool]] = None,
              create: bool = False, **ring_kw) -> int:
    """Driver-side loop over the shared-memory ring; returns the number of operations served. Ends when
    the channel is closed, on a `shutdown` control operation, or when `stop()` turns true."""
    from .._C import pie_host
    ring = pie_host.ShmChannel(name, create, ring_kw.get("slots", 64), ring_kw.get("req_capacity", 8 << 20),
                               ring_kw.get("resp_capacity", 8 << 20), abi.SCHEMA_VERSION, _schema_hash64(),
                               ring_kw.get("spin_iters", 2000))
    served = 0
    while not (stop and stop()):
        try:
            got = ring.next_request(idle_timeout_s)
        except RuntimeError:
            break                                # closed
        if got is None:
            continue
        slot, _req_id, buf = got
        shutdown = False
        try:
            kind = abi.frame_kind(buf)
            if kind == abi.KIND_FORWARD_REQUEST:
                resp = driver.fire_batch(abi.unpack_forward_request(buf))
                out = (abi.pack_tokens(resp.tokens, resp.t_forward_us, resp.t_total_us) if resp.tokens is not None
                       and resp.spec_accepted is None and all(s.kind == "token" for s in resp.slots)
                       else abi.pack_forward_response(resp))
            elif kind == abi.KIND_DECODE_STEP:
                step, parity = abi.unpack_decode_step(buf)
                out = abi.pack_tokens(driver.decode_async(step, parity).wait())
            elif kind == abi.KIND_COPY_REQUEST:
                driver.copy(abi.unpack_copy_request(buf))
                out = abi.pack_control({"value": None})
            else:
                msg = abi.unpack_control(buf)
                shutdown = msg.get("op") == "shutdown"
                out = abi.pack_control({"value": dispatch(driver, OP_CONTROL, msg)})
        except Exception as e:  # noqa: BLE001 - reported to the caller, the loop goes on
            out = abi.pack_control({"error": f"{type(e).__name__}: {e}"})
        ring.respond(slot, out)
        served += 1
        if shutdown:
            break
    return served


# ----------------------------------------------------------------------------- the proxy
class _Waiter:
    def __init__(self, ticket, timeout):
        self.ticket, self.timeout = ticket, timeout

    def wait(self) -> np.ndarray:
        return self.ticket.result(self.timeout)


class ChannelDriver:
    """A driver behind a channel: the protocol the engine uses (capabilities, fire_batch, decode_async,
    copy, adapter operations, health, shutdown), each call one operation on the channel."""

    def __init__(self, channel, timeout_s: float = 120.0, on_shutdown: Optional[Callable[[], None]] = None):
        self.channel, self.timeout_s, self._on_shutdown = channel, timeout_s, on_shutdown
        self._caps: Optional[Capabilities] = None
        self.alive = True

    def _control(self, op: str, *args):
        return self.channel.submit_sync(OP_CONTROL, {"op": op, "args": list(args)}, self.timeout_s)

    def capabilities(self) -> Capabilities:
        if self._caps is None:
            self._caps = Capabilities(**self._control("caps"))
        return self._caps

    def fire_batch(self, req: ForwardRequest) -> ForwardResponse:
        return self.channel.submit_sync(OP_FORWARD, req, self.timeout_s)

    def decode_async(self, step, parity: int):
        return _Waiter(self.channel.submit(OP_DECODE, (step, parity)), self.timeout_s)

    def copy(self, req: CopyRequest) -> None:
        self.channel.submit_sync(OP_COPY, req, self.timeout_s)

    def health(self) -> bool:
        if not self.alive:
            return False
        try:
            return bool(self.channel.submit_sync(OP_CONTROL, {"op": "health"}, 5.0))
        except Exception:  # noqa: BLE001
            return False

    def create_adapter(self, *a):
        return self._control("create_adapter", *a)

    def destroy_adapter(self, *a):
        return self._control("destroy_adapter", *a)

    def fork_adapter(self, *a):
        return self._control("fork_adapter", *a)

    def save_adapter(self, *a):
        return self._control("save_adapter", *a)

    def load_adapter(self, *a):
        return self._control("load_adapter", *a)

    def zo_apply(self, *a):
        return self._control("zo_apply", *a)

    def copy_rs(self, src_slot: int, dst_slot: int):
        return self._control("copy_rs", int(src_slot), int(dst_slot))

    def put_media(self, slot: int, kind: str, patches, grids) -> int:
        p = np.ascontiguousarray(patches, dtype=np.float16)
        return self._control("put_media", int(slot), kind, base64.b64encode(p.tobytes()).decode(), list(p.shape),
                             [[int(x) for x in g] for g in grids])

    def release_media(self, slot: int):
        return self._control("release_media", int(slot))

    def shutdown(self) -> None:
        if self.alive:
            self.alive = False
            try:
                self.channel.submit_sync(OP_CONTROL, {"op": "shutdown"}, 5.0)
            except Exception:  # noqa: BLE001
                pass
            self.channel.close()
            if self._on_shutdown:
                self._on_shutdown()


def make_channel(driver, profile: str = "inproc"):
    """`inproc` (blocking), `latency` (polling) - the two in-process profiles of the configuration."""
    if profile in ("latency", "polling"):
        return PollingChannel(driver)
    if profile in ("inproc", "blocking", ""):
        return InProcChannel(driver)
    raise ValueError(f"unknown channel profile {profile!r}")


def spawn_driver_process(name: str, model_section: dict, ready_timeout_s: float = 600.0):
    """Start `python -m pie_b200.driver.channel --serve NAME` for one `[[model]]` table (as a dict) and
    return (ChannelDriver, Popen). The runtime owns the shared segment; the child ends with its parent."""
    import json
    import subprocess
    import sys
    ch = ShmemChannel(name, create=True)
    proc = subprocess.Popen([sys.executable, "-m", "pie_b200.driver.channel", "--serve", name,
                             "--model-json", json.dumps(model_section)])

    def reap():
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            proc.kill()
    drv = ChannelDriver(ch, on_shutdown=reap)
    deadline = time.monotonic() + ready_timeout_s
    while True:                                   # the first answer is the ready signal: capabilities
        if proc.poll() is not None:
            ch.close()
            raise RuntimeError(f"driver process exited with {proc.returncode} before it was ready")
        try:
            drv._caps = Capabilities(**ch.submit_sync(OP_CONTROL, {"op": "caps"}, 2.0))
            return drv, proc
        except ChannelTimeout:
            if time.monotonic() > deadline:
                proc.kill()
                raise


def _main(argv=None) -> int:
    import argparse
    import json
    ap = argparse.ArgumentParser(description="serve one model's driver over a shared-memory channel")
    ap.add_argument("--serve", required=True, help="name of the shared segment (created by the runtime)")
    ap.add_argument("--model-json", required=True, help="the [[model]] table of the configuration, as JSON")
    a = ap.parse_args(argv)
    from ..server import config as cfgmod
    from ..server.serve import _build_drivers_direct
    sec = cfgmod._build(cfgmod.ModelSection, json.loads(a.model_json), "model")
    drivers, _, _, _ = _build_drivers_direct(sec)
    ppid = os.getppid()
    serve_shm(drivers[0], a.serve, stop=lambda: os.getppid() != ppid)
    return 0


if __name__ == "__main__":
    raise SystemExit(_main())
