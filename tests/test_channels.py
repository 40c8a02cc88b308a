"""Runtime <-> driver channels: blocking in-process, polled ring, shared memory to another process; the
driver proxy over each; abort, timeout and slot-reuse behaviour (runtime/src/driver/{inproc,inproc_polling,
shmem}.rs, driver/bridge/src/ipc.rs)."""
import json
import multiprocessing as mp
import os
import threading
import time

import numpy as np
import pytest

from pie_b200.driver import abi, channel as ch
from pie_b200.driver.executor import CohortStep
from pie_b200.driver.mock import CounterBehavior, DelayedBehavior, FailAfterBehavior, MockDriver
from pie_b200.driver.schema import CopyDir, CopyRequest, ForwardRequest, SamplerKind, SamplerSpec


def _req(first=5, n=3, samplers=None):
    i32 = lambda *a: np.asarray(a, dtype=np.int32)
    return ForwardRequest(tokens=np.arange(first, first + n, dtype=np.int32), positions=np.arange(n, dtype=np.int32),
                          qo_indptr=i32(0, n), kv_page_indices=i32(0), kv_page_indptr=i32(0, 1), kv_last_page_lens=i32(n),
                          slot_req=i32(0), slot_row=i32(n - 1), slot_samplers=samplers or [SamplerSpec()])


def _step(r=2):
    z = lambda dt: np.zeros(r, dt)
    return CohortStep(r, np.asarray([7, 9], np.int32), np.full(r, -1, np.int32), np.asarray([3, 4], np.int32),
                      np.asarray([4, 5], np.int32), np.asarray([0, 1, 2], np.int32), np.asarray([0, 1], np.int32),
                      np.ones(r, np.float32), z(np.int32), np.ones(r, np.float32), z(np.float32), np.asarray([1, 2], np.int64))


@pytest.mark.parametrize("kind", ["inproc", "latency"])
def test_in_process_channels_carry_every_operation(kind):
    drv = MockDriver(CounterBehavior(), total_pages=77)
    c = ch.make_channel(drv, kind)
    proxy = ch.ChannelDriver(c)
    assert proxy.capabilities().total_pages == 77
    assert proxy.fire_batch(_req()).slots[0].token == 8
    assert proxy.decode_async(_step(), 0).wait().tolist() == [8, 10]
    proxy.copy(CopyRequest(CopyDir(0), np.asarray([1], np.int32), np.asarray([2], np.int32)))
    assert len(drv.recorder.copies) == 1 and proxy.health()
    # many producers: every request gets its own answer
    out = {}

    def worker(k):
        out[k] = [proxy.fire_batch(_req(first=100 * k + j)).slots[0].token for j in range(20)]
    ts = [threading.Thread(target=worker, args=(k,)) for k in range(8)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert all(out[k] == [100 * k + j + 3 for j in range(20)] for k in range(8))
    proxy.shutdown()
    assert not proxy.health()
    with pytest.raises(ch.ChannelClosed):
        c.submit(ch.OP_FORWARD, _req()).result(1.0)


def test_driver_errors_travel_back_and_abort_fails_the_queue():
    drv = MockDriver(FailAfterBehavior(CounterBehavior(), 1))
    c = ch.InProcChannel(drv)
    assert c.submit_sync(ch.OP_FORWARD, _req()).slots[0].token == 8
    with pytest.raises(RuntimeError):
        c.submit_sync(ch.OP_FORWARD, _req())
    slow = ch.InProcChannel(MockDriver(DelayedBehavior(CounterBehavior(), 0.2)))
    t1 = slow.submit(ch.OP_FORWARD, _req())
    t2 = slow.submit(ch.OP_FORWARD, _req())
    time.sleep(0.05)
    slow.abort("driver lost")
    with pytest.raises(ch.ChannelClosed, match="driver lost"):
        t2.result(2.0)
    assert t1.result(2.0).slots[0].token == 8            # the one being served finishes
    with pytest.raises(ch.ChannelTimeout):
        ch.InProcChannel(MockDriver(DelayedBehavior(CounterBehavior(), 0.3))).submit(ch.OP_FORWARD, _req()).result(0.01)
    c.close()
    slow.close()


def test_priority_orders_the_blocking_queue():
    drv = MockDriver(DelayedBehavior(CounterBehavior(), 0.05))
    c = ch.InProcChannel(drv)
    c.submit(ch.OP_FORWARD, _req(n=1))                            # occupies the service thread
    time.sleep(0.01)
    late = c.submit(ch.OP_FORWARD, _req(n=2), priority=5)
    urgent = c.submit(ch.OP_FORWARD, _req(n=3), priority=0)
    late.result(5.0), urgent.result(5.0)
    assert [f["tokens"] for f in drv.recorder.fires] == [1, 3, 2]
    c.close()


def test_polling_ring_wraps_and_parks_when_idle():
    drv = MockDriver(CounterBehavior())
    c = ch.PollingChannel(drv, slots=8, spin_budget=50)
    for j in range(40):                                             # five laps of the ring
        assert c.submit_sync(ch.OP_FORWARD, _req(first=j), 5.0).slots[0].token == j + 3
    time.sleep(0.1)
    assert c.parks >= 1 and c.served == 40
    assert c.submit_sync(ch.OP_FORWARD, _req(first=1), 5.0).slots[0].token == 4      # wakes from the park
    c.close()


def _serve_child(name, fail_after=None, delay=0.0):
    beh = CounterBehavior()
    if delay:
        beh = DelayedBehavior(beh, delay)
    if fail_after is not None:
        beh = FailAfterBehavior(beh, fail_after)
    ch.serve_shm(MockDriver(beh, total_pages=55), name)


def test_shared_memory_channel_to_a_driver_process():
    name = f"pie_b200_test_ch_{os.getpid()}"
    c = ch.ShmemChannel(name, create=True, slots=4, req_capacity=1 << 16, resp_capacity=1 << 20, timeout_s=20.0)
    ctx = mp.get_context("spawn")
    p = ctx.Process(target=_serve_child, args=(name, 39))
    p.start()
    try:
        proxy = ch.ChannelDriver(c, timeout_s=20.0)
        assert proxy.capabilities().total_pages == 55
        r = proxy.fire_batch(_req())
        assert r.slots[0].token == 8 and r.tokens.tolist() == [8]                      # token fast path
        r = proxy.fire_batch(_req(samplers=[SamplerSpec(SamplerKind.DIST, top_k=2)]))
        assert r.slots[0].kind == "distribution" and r.slots[0].ids == [8, 9]         # full response frame
        assert proxy.decode_async(_step(), 1).wait().tolist() == [8, 10]
        proxy.copy(CopyRequest(CopyDir(0), np.asarray([1], np.int32), np.asarray([2], np.int32)))
        assert c.last_service_us > 0 and proxy.health()
        # more requests in flight than slots, from several threads
        out = {}

        def worker(k):
            out[k] = [proxy.fire_batch(_req(first=100 * k + j)).slots[0].token for j in range(6)]
        ts = [threading.Thread(target=worker, args=(k,)) for k in range(6)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        assert all(out[k] == [100 * k + j + 3 for j in range(6)] for k in range(6))
        with pytest.raises(RuntimeError, match="driver"):                               # the 40th fire fails in the child
            proxy.fire_batch(_req())
        assert proxy.health()                                                           # and the loop goes on
        proxy.shutdown()
        p.join(timeout=20)
        assert p.exitcode == 0
    finally:
        if p.is_alive():
            p.kill()


def test_shared_memory_timeout_frees_the_slot_and_schema_mismatch_is_refused():
    from pie_b200._C import pie_host
    name = f"pie_b200_test_ch2_{os.getpid()}"
    c = ch.ShmemChannel(name, create=True, slots=2, req_capacity=1 << 12, resp_capacity=1 << 12, timeout_s=5.0)
    with pytest.raises(RuntimeError, match="wire schema"):
        pie_host.ShmChannel(name, False, 0, 0, 0, abi.SCHEMA_VERSION, 12345, 10)
    with pytest.raises(ch.ChannelTimeout):                                             # nobody serves
        c.submit(ch.OP_CONTROL, {"op": "health"}).result(0.05)
    with pytest.raises(ch.ChannelTimeout):
        c.submit(ch.OP_CONTROL, {"op": "health"}).result(0.05)
    stop = {"v": False}
    t = threading.Thread(target=lambda: ch.serve_shm(MockDriver(CounterBehavior()), name, idle_timeout_s=0.05,
                                                     stop=lambda: stop["v"]))
    t.start()
    try:
        # both slots were abandoned: the server frees them instead of answering, and new work goes through
        assert c.submit_sync(ch.OP_CONTROL, {"op": "health"}, 5.0) is True
        assert [c.ring.slot_state(i) for i in range(2)] == [0, 0]
        with pytest.raises(ValueError):
            c.ring.submit(b"x" * (1 << 13))                                            # larger than a slot
    finally:
        stop["v"] = True
        t.join(timeout=5)
    c.close()
    with pytest.raises(ch.ChannelClosed):
        c.submit(ch.OP_CONTROL, {"op": "health"})


@pytest.mark.parametrize("ipc", ["inproc", "latency", "shmem"])
def test_engine_generates_the_same_tokens_over_every_channel(ipc, tmp_path):
    """The serving stack with `[model.driver] ipc = ...`: same greedy tokens as the direct call."""
    from pie_b200.server import config as cfgmod
    from pie_b200.server.serve import start_engine

    def run(kind):
        cfg = cfgmod.parse(f'[auth]\nenabled = false\n[[model]]\nname = "m"\npreset = "tiny-llama"\n'
                           f'[model.driver]\ntype = "cpu"\nipc = "{kind}"\n')
        h = start_engine(cfg, serve=False)
        try:
            out = [json.loads(h.engine.run("text-completion", {"prompt_tokens": p, "max_tokens": 6, "temperature": 0.0,
                                                              "stop_tokens": []}, 120))["tokens"]
                   for p in ([1, 2, 3, 4, 5], [9, 8, 7])]
            st = h.engine.model_status()["models"]["m"]
            assert st["kv_pages_used"] == 0
        finally:
            h.shutdown()
        return out
    assert run(ipc) == run("direct")
