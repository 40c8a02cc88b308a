"""Allocation order of the context manager under contention: priority gate, eviction by rank, deferral,
the restore queue with its wake-ups, restore admission and data-parallel placement
(runtime/src/context/sched.rs:367-417, :717-868, :881-938; scenarios after sched.rs:1196+)."""
import pytest

from pie_b200.runtime.context import ContextError, ContextManager, Deferred, State
from pie_b200.runtime.pagestore import PageStore

PS = 4


def mgr(pages=8, drivers=1, swap=0):
    return ContextManager("m", PS, [PageStore(pages) for _ in range(drivers)], swap_pages=swap)


def fill(m, cid, n_tokens, commit=True, start=0):
    m.reserve_working_pages(cid, -(-n_tokens // PS))
    m.append_working_tokens(cid, list(range(start, start + n_tokens)), list(range(n_tokens)))
    if commit:
        m.commit_working_pages(cid, n_tokens // PS)


def test_eviction_only_takes_contexts_the_requester_does_not_rank_below():
    m = mgr(pages=4)
    rich, poor = m.create("rich"), m.create("poor")
    m.set_bid(rich, 5.0)
    m.set_bid(poor, 1.0)
    fill(m, rich, 8, commit=False)
    fill(m, poor, 8, commit=False)
    assert m.stores[0].pool.free_count == 0
    with pytest.raises(Deferred):
        m.reserve_working_pages(poor, 1)               # would have to evict `rich`
    assert m.contexts[rich].state == State.ACTIVE and m.counters["deferred"] == 1
    m.reserve_working_pages(rich, 1)                   # evicts `poor`
    assert m.contexts[poor].state == State.SUSPENDED and m.counters["evictions"] == 1
    assert issubclass(Deferred, ContextError)


def test_equal_bids_evict_newest_first_as_before():
    m = mgr(pages=4)
    a, b, c = m.create("a"), m.create("b"), m.create("c")
    fill(m, a, 8, commit=False)
    fill(m, b, 8, commit=False)
    m.reserve_working_pages(c, 1)
    assert m.contexts[b].state == State.SUSPENDED and m.contexts[a].state == State.ACTIVE


def test_priority_gate_holds_free_pages_for_the_queue_head():
    m = mgr(pages=6)
    vip, low, other = m.create("vip"), m.create("low"), m.create("other")
    m.set_bid(vip, 9.0)
    fill(m, vip, 16, commit=False)                     # 4 pages
    m.suspend(vip)                                     # no swap tier: dropped, needs 4 pages to return
    fill(m, other, 12, commit=False)                   # 3 pages used, 3 free
    pin = m.pin(other, 0)
    woke = []
    m.when_restorable(vip, lambda: woke.append("vip"))
    assert woke == [] and m.restore_queue[0]           # cannot return: only 3 free and `other` is pinned
    with pytest.raises(Deferred, match="held for context"):
        m.reserve_working_pages(low, 1)                # the 3 free pages are spoken for
    assert m.counters["gate_holds"] == 1
    m.set_bid(low, 10.0)
    m.reserve_working_pages(low, 1)                    # outranks the head: served
    m.release_working_pages(low, 1)
    assert woke == []
    m.unpin(other)                                     # now evictable -> the head can come back
    assert woke == ["vip"] and not m.restore_queue[0] and m.counters["restore_wakeups"] == 1
    assert m.restore(vip) and m.contexts[vip].state == State.ACTIVE
    assert pin.context_id == other


def test_restore_queue_is_ordered_by_rank_then_arrival_and_drains_on_destroy():
    m = mgr(pages=4)
    ids = [m.create(f"o{i}") for i in range(3)]
    for cid, bid in zip(ids, (1.0, 3.0, 1.0)):
        m.set_bid(cid, bid)
        fill(m, cid, 8, commit=False)                  # each needs 2 pages; the third evicts the first ...
    hog = m.create("hog")
    m.set_bid(hog, 50.0)
    fill(m, hog, 16, commit=False)                     # ... and the hog evicts everybody
    assert all(m.contexts[c].state == State.SUSPENDED for c in ids)
    m.pin(hog, 0)
    order = []
    for cid in ids:
        m.when_restorable(cid, lambda c=cid: order.append(c))
    assert [e[0] for e in m.restore_queue[0]] == [ids[1], ids[0], ids[2]]
    assert not m.can_restore(ids[1])
    with pytest.raises(Deferred):
        m.restore(ids[1])
    m.unpin(hog)
    m.destroy(hog)
    assert order[0] == ids[1] and set(order) == set(ids)      # all fit once the hog is gone (4 free, 2 each: two at a time)


def test_can_restore_respects_the_utilization_pause_only_while_others_run():
    m = mgr(pages=10)
    a, b = m.create("a"), m.create("b")
    fill(m, a, 8, commit=False)
    m.suspend(a)
    fill(m, b, 28, commit=False)                       # 7 of 10 pages used; a's return makes 9 > 8.5
    assert m.can_restore(a)                            # nobody is pinned: the pool is idle, come back
    m.pin(b, 0)
    assert not m.can_restore(a)                        # a running batch: stay under the pause threshold
    m.restore_pause_at_utilization = 0.95
    assert m.can_restore(a)


def test_best_driver_prefers_the_replica_that_already_holds_the_prefix():
    m = mgr(pages=8, drivers=2)
    c0 = m.create("a", driver=1)
    fill(m, c0, 8)                                     # two committed pages on replica 1
    chain = list(m.contexts[c0].chain)
    filler = m.create("f", driver=1)
    fill(m, filler, 12, commit=False, start=100)       # replica 1 is also the fuller one
    assert m.least_loaded_driver() == 0
    assert m.best_driver_for(chain) == 1               # but the prefix is there
    assert m.best_driver_for([], n_pages=2) == 0       # nothing to reuse: most free pages
    assert m.best_driver_for([123, 456]) == 0          # unknown chain: same


def test_deferred_forward_waits_in_the_queue_and_runs_after_pages_return():
    import json
    import threading
    from test_runtime_cpu import CounterBehavior, MockDriver, engine_with
    eng = engine_with(MockDriver(CounterBehavior(), total_pages=70, page_size=16))
    try:
        entry = eng.models["mock"]
        m = entry.ctxm
        hog = m.create("hog")
        m.set_bid(hog, 99.0)
        m.reserve_working_pages(hog, 68)
        m.pin(hog, 0)                                  # 68 of 70 pages pinned by a context that outranks everyone
        done = {}

        def run():
            done["out"] = json.loads(eng.run("text-completion", {"prompt_tokens": list(range(40)), "max_tokens": 3,
                                                                 "stop_tokens": [], "per_step": True}, 60))
        t = threading.Thread(target=run)
        t.start()
        t.join(timeout=1.5)
        assert t.is_alive()                            # needs 3 pages, 2 free: parked, not failed
        m.unpin(hog)
        m.destroy(hog)
        t.join(timeout=30)
        assert not t.is_alive() and done["out"]["tokens"] == [40, 41, 42]
    finally:
        eng.shutdown()
