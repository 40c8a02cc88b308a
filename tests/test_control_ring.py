"""Host control plane of tensor parallelism: rank 0 publishes steps into a shared-memory ring,
follower processes consume them in order (CPU only, real processes)."""
import multiprocessing as mp
import os
import time

import numpy as np

from pie_b200.parallel.comm import KIND_BATCH, KIND_DECODE, KIND_STOP, StepRing


def _follower(name, world, rank, q):
    ring = StepRing(name, world, rank, cap=1 << 16, create=False)
    got = []
    while True:
        kind, payload, meta = ring.receive(timeout=30)
        if kind == KIND_STOP:
            ring.ack()
            break
        got.append((kind, int(payload.view(np.int32).sum()) if len(payload) else 0, meta[0]))
        ring.ack()
    ring.close()
    q.put((rank, got))


def test_ring_delivers_every_step_in_order_to_every_follower():
    name = f"pie_b200_test_ring_{os.getpid()}"
    world = 3
    ring = StepRing(name, world, 0, cap=1 << 16, create=True)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_follower, args=(name, world, r, q)) for r in range(1, world)]
    for p in procs:
        p.start()
    want = []
    try:
        for i in range(50):
            data = np.arange(i + 1, dtype=np.int32)
            kind = KIND_DECODE if i % 2 else KIND_BATCH
            ring.publish(kind, data, (i,))
            want.append((kind, int(data.sum()), i))
        ring.publish(KIND_STOP, None)
        res = dict(q.get(timeout=60) for _ in procs)
    finally:
        for p in procs:
            p.join(timeout=10)
        ring.close(unlink=True)
    assert res[1] == want and res[2] == want


def _stalling_follower(name, world, rank, consume, exit_after):
    """Consumes `consume` steps, then either exits (exit_after) or stops acknowledging."""
    ring = StepRing(name, world, rank, cap=1 << 12, create=False)
    for _ in range(consume):
        ring.receive(timeout=30)
        ring.ack()
    if not exit_after:
        time.sleep(20)
    ring.close()


def _run_leader_against(follower_args, ack_timeout_s):
    import pytest
    name = f"pie_b200_test_ring_f_{os.getpid()}_{int(time.time() * 1e3) & 0xFFFF}"
    ring = StepRing(name, 2, 0, cap=1 << 12, create=True, ack_timeout_s=ack_timeout_s)
    ctx = mp.get_context("spawn")
    p = ctx.Process(target=_stalling_follower, args=(name, 2, 1, *follower_args))
    p.start()
    t0 = time.time()
    try:
        with pytest.raises(RuntimeError) as ei:
            for i in range(64):
                ring.publish(KIND_BATCH, np.arange(4, dtype=np.int32), (i,))
        return str(ei.value), time.time() - t0
    finally:
        p.kill()
        p.join(timeout=10)
        ring.close(unlink=True)


def test_publish_fails_fast_when_a_follower_exits():
    msg, dt = _run_leader_against((3, True), ack_timeout_s=60)
    assert "exited" in msg and dt < 30


def test_publish_gives_up_on_a_follower_that_stops_acknowledging():
    msg, dt = _run_leader_against((3, False), ack_timeout_s=1.0)
    assert "stopped consuming" in msg and dt < 15


def _orphan_follower(name, q):
    ring = StepRing(name, 2, 1, cap=1 << 12, create=False)
    try:
        ring.receive(timeout=60)
        q.put("got a step")
    except TimeoutError as e:
        q.put(str(e))
    ring.close()


def _short_lived_leader(name, ready):
    ring = StepRing(name, 2, 0, cap=1 << 12, create=True)
    ready.put(1)
    time.sleep(1.0)
    os._exit(0)      # dies without publishing or unlinking


def test_follower_notices_a_dead_leader():
    name = f"pie_b200_test_ring_o_{os.getpid()}"
    ctx = mp.get_context("spawn")
    ready, q = ctx.Queue(), ctx.Queue()
    leader = ctx.Process(target=_short_lived_leader, args=(name, ready))
    leader.start()
    ready.get(timeout=30)
    f = ctx.Process(target=_orphan_follower, args=(name, q))
    f.start()
    try:
        assert "rank 0 exited" in q.get(timeout=40)
    finally:
        leader.join(timeout=5)
        f.join(timeout=5)
        from multiprocessing import shared_memory
        try:
            shm = shared_memory.SharedMemory(name=name)
            shm.close()
            shm.unlink()
        except FileNotFoundError:
            pass
