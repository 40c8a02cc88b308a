"""Host runtime on a CPU with scripted mock drivers: page store, contexts, scheduler limits,
chunked prefill, failure delivery, market. Mirrors the reference's strategy of testing every
scheduler / KV / market path against a mock driver channel (runtime/tests/common/mock_device.rs)."""
import json
import threading
import time

import numpy as np
import pytest

from pie_b200.driver.mock import (CallRecorder, CounterBehavior, DelayedBehavior, DummyDriver, FailAfterBehavior,
                                  MockDriver)
from pie_b200.driver.schema import Capabilities, SamplerSpec
from pie_b200.inferlets import install_all
from pie_b200.runtime import brle, pagestore
from pie_b200.runtime.context import ContextError, ContextManager
from pie_b200.runtime.engine import Engine, EngineConfig
from pie_b200.runtime.market import Market
from pie_b200.runtime.scheduler import BatchAccumulator, BatchScheduler, PendingRequest, fold


# ------------------------------------------------------------------ BRLE
def test_brle_roundtrip_and_ops():
    rng = np.random.default_rng(0)
    for _ in range(200):
        n = int(rng.integers(0, 300))
        a, b = rng.random(n) < 0.4, rng.random(n) < 0.6
        ra, rb = brle.encode(a), brle.encode(b)
        assert (brle.decode(ra, n) == a).all()
        assert (brle.decode(brle.logical_and(ra, rb), n) == (a & b)).all()
        assert brle.count_true(ra) == int(a.sum())
    assert brle.range_mask(10, 2, 5) == [2, 3, 5]
    assert brle.all_true(7) == [0, 7]
    drop = brle.droppable_pages([[16, 16, 32], [40, 8]], 16, 4)
    assert list(drop) == [True, False, False, True]


# ------------------------------------------------------------------ page store (both implementations)
@pytest.mark.parametrize("impl", ["python", "native"])
def test_pagestore_dedup_share_release(impl):
    if impl == "native" and not pagestore.NATIVE:
        pytest.skip("native host module not built")
    Store = pagestore.PyPageStore if impl == "python" else pagestore.PageStore
    hash_fn = pagestore.py_page_hash if impl == "python" else pagestore.page_hash
    s = Store(8)
    p = s.pool.alloc(4)
    h1 = hash_fn(0, [1, 2, 3], [0, 1, 2])
    h2 = hash_fn(h1, [4, 5, 6], [3, 4, 5])
    assert hash_fn(0, [1, 2, 3], [0, 1, 2]) == h1 and hash_fn(0, [1, 2, 4], [0, 1, 2]) != h1
    assert s.extend(0, h1, p[0]) == (p[0], False)
    assert s.extend(h1, h2, p[1]) == (p[1], False)
    # a second context commits the same content: deduplicated onto the existing pages
    assert s.extend(0, h1, p[2]) == (p[0], True)
    s.pool.free([p[2]])
    assert s.prefix_len([h1, h2, 12345]) == 2
    assert s.physical_ids([h1, h2]) == [p[0], p[1]]
    assert abs(s.effective_pages([h1, h2], 1) - (1 + 0.5 + 1.0)) < 1e-9
    assert s.release([h1]) == []                  # still held by the first chain
    assert sorted(s.release([h1, h2])) == sorted([p[0], p[1]])
    assert s.pool.free_count == 7
    s.pool.free([p[3], p[3]])                      # double free is detected, not fatal
    assert s.pool.double_free_count == 1 and s.pool.free_count == 8


# ------------------------------------------------------------------ contexts
def make_ctxm(pages=16, swap=0, copies=None):
    copies = copies if copies is not None else []
    return ContextManager("m", 4, [pagestore.PageStore(pages)], lambda d, r: copies.append(r), swap_pages=swap), copies


def fill(cm, cid, toks, start):
    need = -(-(cm.kv_len(cid) + len(toks)) // 4) - cm.committed_page_count(cid) - cm.working_page_count(cid)
    if need > 0:
        cm.reserve_working_pages(cid, need)
    cm.append_working_tokens(cid, toks, list(range(start, start + len(toks))))


def test_context_commit_fork_dedup_and_audit():
    cm, copies = make_ctxm()
    a = cm.create("p1")
    fill(cm, a, list(range(10)), 0)
    cm.commit_working_pages(a, 2)
    assert cm.committed_page_count(a) == 2 and cm.working_page_token_count(a) == 2
    b = cm.fork(a, owner="p2")
    assert len(copies) == 1 and copies[0].direction.name == "D2D"     # only working pages are copied
    assert cm.kv_len(b) == 10 and cm.pages_used() == 4                # 2 shared + 1 working each
    # same content committed from scratch by a third context lands on the shared pages
    c = cm.create("p3")
    fill(cm, c, list(range(8)), 0)
    cm.commit_working_pages(c, 2)
    assert cm.counters["dedup_pages"] == 2 and cm.pages_used() == 4
    cm.audit()
    with pytest.raises(ContextError):
        cm.pin(a, 100)                                                # KV invariant
    pinned = cm.pin(a, 2)
    assert pinned.kv_len == 10 and len(pinned.pages) == 3
    cm.unpin(a)
    for x in (a, b, c):
        cm.destroy(x)
    assert cm.pages_used() == 0
    cm.audit()


def test_commit_requires_increasing_positions():
    cm, _ = make_ctxm()
    a = cm.create("p")
    cm.reserve_working_pages(a, 1)
    cm.append_working_tokens(a, [1, 2, 3, 4], [0, 1, 1, 2])
    with pytest.raises(ContextError):
        cm.commit_working_pages(a, 1)


def test_snapshots_save_open_take_delete():
    cm, _ = make_ctxm()
    a = cm.create("p1")
    fill(cm, a, list(range(6)), 0)
    cm.save(a, "alice", "s1")
    cm.destroy(a)
    b = cm.open("alice", "s1", "p2")
    assert cm.kv_len(b) == 6
    with pytest.raises(ContextError):
        cm.open("bob", "s1", "p3")                                    # snapshots are per user
    c = cm.take("alice", "s1", "p3")
    assert cm.contexts[c].owner == "p3"
    with pytest.raises(ContextError):
        cm.open("alice", "s1", "p4")                                  # taken
    name = cm.snapshot(b, "alice")
    cm.delete_snapshot("alice", name)
    cm.destroy_owner("p2"); cm.destroy_owner("p3")
    assert cm.pages_used() == 0


def test_truncate_release_and_eviction_restore_with_swap():
    cm, copies = make_ctxm(pages=6, swap=4)
    a = cm.create("p1")
    fill(cm, a, list(range(7)), 0)
    cm.truncate_working_page_tokens(a, 2)
    assert cm.kv_len(a) == 5
    cm.release_working_pages(a, 1)
    assert cm.kv_len(a) == 4 and cm.working_page_count(a) == 1
    # fill the pool from a second process: the first context is evicted (stashed on the CPU tier)
    b = cm.create("p2")
    cm.set_bid(a, 0.1)
    cm.reserve_working_pages(b, 6)
    assert cm.contexts[a].state.value == "suspended" and cm.counters["evictions"] == 1
    assert any(r.direction.name == "D2H" for r in copies)
    cm.release_working_pages(b, 6)
    replay = cm.restore(a)
    assert replay == [] and any(r.direction.name == "H2D" for r in copies)    # came back from the stash
    assert cm.kv_len(a) == 4
    cm.audit()


def test_eviction_without_swap_needs_replay():
    cm, _ = make_ctxm(pages=4, swap=0)
    a = cm.create("p1")
    fill(cm, a, list(range(6)), 0)
    cm.commit_working_pages(a, 1)
    b = cm.create("p2")
    cm.reserve_working_pages(b, 4)
    assert cm.contexts[a].state.value == "suspended"
    cm.release_working_pages(b, 4)
    replay = cm.restore(a)
    # committed page was freed with the eviction: both spans must be recomputed
    assert [(len(t), first) for t, _, first in replay] == [(4, 0), (2, 4)]


# ------------------------------------------------------------------ scheduler
def req(cid, n, kv=0, pages=None, samplers=True):
    pages = pages or list(range(-(-(kv + n) // 16)))
    return PendingRequest(cid, list(range(n)), list(range(kv, kv + n)), pages, kv,
                          [(n - 1, SamplerSpec.greedy())] if samplers else [])


def test_accumulator_enforces_driver_limits():
    caps = Capabilities(total_pages=100, kv_page_size=16, max_forward_requests=3, max_forward_tokens=40,
                        max_page_refs=5, max_sampler_rows=2, max_logit_rows=2)
    acc = BatchAccumulator(caps, 16)
    assert acc.fits(req(1, 16)); acc.push(req(1, 16))
    assert acc.fits(req(2, 16)); acc.push(req(2, 16))
    assert not acc.fits(req(3, 16))                       # tokens 48 > 40 (and sampler rows 3 > 2)
    assert not acc.fits(req(3, 1, samplers=True))         # sampler rows
    assert acc.fits(req(3, 1, samplers=False))
    acc.push(req(3, 1, samplers=False))
    assert not acc.fits(req(4, 1, samplers=False))        # requests
    assert len(acc.take()) == 3 and acc.usage.tokens == 0
    acc.push(req(5, 1, kv=79, pages=list(range(5))))
    assert not acc.fits(req(6, 1, kv=0, samplers=False))  # page refs 5 + 1 > 5


def test_accumulator_counts_logit_and_prob_rows_after_the_compact_projection():
    """Eight limits: logit rows and probability rows are distinct token rows, not sampler slots, and the
    label and mask-byte budgets hold too (scheduler.rs:728-980)."""
    from pie_b200.driver.schema import SamplerKind
    caps = Capabilities(total_pages=100, kv_page_size=16, max_forward_requests=10, max_forward_tokens=100,
                        max_sampler_rows=8, max_logit_rows=3, max_prob_rows=1, max_logprob_labels=4,
                        max_custom_mask_bytes=64)
    acc = BatchAccumulator(caps, 16)
    probes = PendingRequest(1, [1, 2, 3, 4], [0, 1, 2, 3], [0], 0,
                            [(3, SamplerSpec.greedy()), (3, SamplerSpec(SamplerKind.DIST, top_k=5)),
                             (3, SamplerSpec(SamplerKind.ENTROPY)), (3, SamplerSpec(SamplerKind.LOGPROBS, labels=(1, 2)))])
    c = acc.cost(probes)
    assert (c.sampler_rows, c.logit_rows, c.prob_rows, c.logprob_labels) == (4, 1, 1, 2)
    acc.push(probes)
    assert acc.fits(req(2, 4))                                            # a second logit row, no probabilities
    acc.push(req(2, 4))
    other_row = PendingRequest(3, [1, 2], [0, 1], [0], 0, [(0, SamplerSpec(SamplerKind.ENTROPY))])
    assert not acc.fits(other_row)                                        # a second probability row
    assert acc.fits(req(4, 1))
    acc.push(req(4, 1))
    assert not acc.fits(req(5, 1))                                        # a fourth logit row
    acc.take()
    many = PendingRequest(6, [1], [0], [0], 0, [(0, SamplerSpec(SamplerKind.LOGPROBS, labels=(1, 2, 3, 4, 5)))])
    assert not acc.fits(many)                                             # labels 5 > 4
    masked = PendingRequest(7, [1] * 8, list(range(8)), [0, 1, 2, 3, 4], 64, masks=[[0, 72]] * 8)
    assert acc.cost(masked).mask_bytes == 8 * 9 and not acc.fits(masked)  # 72 bytes of custom mask > 64


def test_fold_builds_csr_and_rejects_short_page_lists():
    items = [req(1, 5, kv=20), req(2, 1, kv=15)]
    f = fold(items, 16)
    assert f.qo_indptr.tolist() == [0, 5, 6] and f.kv_page_indptr.tolist() == [0, 2, 3]
    assert f.kv_last_page_lens.tolist() == [9, 16] and f.slot_row.tolist() == [4, 5]
    with pytest.raises(ValueError):
        fold([PendingRequest(1, [1] * 20, list(range(20)), [0], 0)], 16)


def run_requests(drv, reqs, caps=None, policy="greedy"):
    sched = BatchScheduler(drv, caps or drv.capabilities(), 16, policy)
    results, ev = {}, threading.Event()

    def done(cid):
        def cb(res):
            results[cid] = res
            if len(results) == len(reqs):
                ev.set()
        return cb
    for r in reqs:
        r.on_done = done(r.context_id)
        sched.submit(r)
    assert ev.wait(20)
    sched.shutdown()
    return results, sched


def test_chunked_prefill_splits_oversized_requests_in_order():
    rec = CallRecorder()
    drv = MockDriver(CounterBehavior(), max_tokens=64, recorder=rec)
    n = 150
    r = PendingRequest(7, list(range(1000, 1000 + n)), list(range(n)), list(range(10)), 0,
                       [(10, SamplerSpec.greedy()), (n - 1, SamplerSpec.greedy())])
    results, sched = run_requests(drv, [r])
    assert [f["tokens"] for f in rec.fires] == [64, 64, 22]
    assert [s.token for s in results[7]] == [1011, 1000 + n]          # slots come back in attach order
    assert sched.stats["chunked_requests"] == 1


def test_batch_failure_reaches_every_request_and_scheduler_survives():
    drv = MockDriver(FailAfterBehavior(CounterBehavior(), 1))
    results, _ = run_requests(drv, [req(1, 4)])
    assert results[1][0].token == 4
    results, _ = run_requests(drv, [req(2, 4), req(3, 2)])
    assert all(isinstance(v, Exception) for v in results.values())


def test_adaptive_policy_batches_a_cohort():
    rec = CallRecorder()
    drv = MockDriver(DelayedBehavior(CounterBehavior(), 0.01), recorder=rec)
    reqs = [req(i, 1, kv=3) for i in range(1, 13)]
    run_requests(drv, reqs, policy="adaptive")
    assert sum(f["requests"] for f in rec.fires) == 12 and len(rec.fires) <= 4


# ------------------------------------------------------------------ engine level: failure detection
def engine_with(drv, **cfg):
    eng = Engine(EngineConfig(watchdog_interval_s=0.05, **cfg))
    eng.add_model("mock", drv)
    install_all(eng)
    return eng


def test_engine_generates_through_mock_driver_and_releases_pages():
    eng = engine_with(MockDriver(CounterBehavior(), total_pages=32))
    try:
        out = json.loads(eng.run("text-completion", {"prompt_tokens": [5, 6, 7], "max_tokens": 6, "stop_tokens": []}, 30))
        assert out["tokens"] == [8, 9, 10, 11, 12, 13]
        assert eng.model_status()["models"]["mock"]["kv_pages_used"] == 0
    finally:
        eng.shutdown()


def test_driver_death_fails_processes_fast():
    drv = MockDriver(DelayedBehavior(CounterBehavior(), 0.02), total_pages=64)
    eng = engine_with(drv)
    try:
        p = eng.launch("text-completion", {"prompt_tokens": [1, 2, 3], "max_tokens": 2000, "stop_tokens": []})
        time.sleep(0.3)
        drv.kill()                                        # host-side failure: the driver stops answering
        t0 = time.time()
        with pytest.raises(RuntimeError):
            eng.wait(p, 10)
        assert time.time() - t0 < 5
        q = eng.launch("text-completion", {"prompt_tokens": [1], "max_tokens": 2, "stop_tokens": []})
        with pytest.raises(RuntimeError):
            eng.wait(q, 10)                               # later submissions fail at once too
    finally:
        eng.shutdown()


def test_dummy_driver_honours_logit_masks():
    drv = DummyDriver(vocab=1000)
    r = PendingRequest(1, [1, 2], [0, 1], [0], 0, [(1, SamplerSpec.greedy())], logit_mask=[100, 5, 895])
    for _ in range(20):
        assert 100 <= drv.fire_batch(fold([r], 16)).slots[0].token < 105


# ------------------------------------------------------------------ market
def test_market_conserves_credits_and_orders_victims():
    m = Market(capacity_pages=100, default_endowment_pages=10, oversubscription=1.0, contention_threshold=0.5)
    assert m.try_admit("a") and m.try_admit("b", 30)
    price = m.tick(used_pages=80, batch=[(1, "a", 2.0, 20.0), (2, "b", 3.0, 5.0)])
    assert price == 2.0 and m.rent_of(1) == 40.0 and m.rent_of(2) == 10.0
    assert m.conservation_error() < 1e-9                  # rent is redistributed as dividends
    assert m.defaulted("a") and not m.defaulted("b")
    assert m.victim_key("a", 5.0, 1) < m.victim_key("b", 0.1, 9)   # defaulted first, whatever the bid
    assert m.tick(used_pages=10, batch=[(1, "a", 2.0, 20.0)]) == 0.0   # no contention, no rent


def test_market_admission_queue_is_fifo_with_drain_barrier():
    m = Market(capacity_pages=10, default_endowment_pages=4, oversubscription=1.0)
    admitted = []
    assert m.try_admit("a") and m.try_admit("b")
    assert not m.try_admit("big", 9, on_admit=lambda: admitted.append("big"))
    assert not m.try_admit("small", 1, on_admit=lambda: admitted.append("small"))   # fits, but queued behind
    m.release("a")
    assert admitted == []                                  # 4 + 9 > 10: the head still blocks
    m.release("b")
    assert admitted == ["big", "small"]
    assert not m.debit_tokens("x", 5) or True
    assert m.try_admit("c", 0, token_budget=3) and m.debit_tokens("c", 2) and not m.debit_tokens("c", 2)
    assert m.budget_exhausted("c")
