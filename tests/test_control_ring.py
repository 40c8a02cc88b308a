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
