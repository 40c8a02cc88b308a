"""Context manager: the KV state that inferlets own and manipulate.

A context = a chain of committed pages (immutable, content-hashed, shared through the page
store) + a tail of working pages (exclusive, partially filled) + the lineage of tokens that
fills them. Inferlets allocate (reserve), commit, fork, truncate, release, save/snapshot,
open/take and destroy contexts; forward passes pin a context to read a consistent page list.

States: ACTIVE (resident), PINNED (in a batch), SUSPENDED (evicted: working pages stashed on
the CPU tier or dropped for replay), plus named snapshots that live outside any process.

Behavioural counterpart of runtime/src/context.rs:311-840 (API), :1549-1981 (create, destroy,
commit with position-monotonicity check :1752-1763, pin :1834-1940), context/snapshot.rs:37-392
(fork / save / open / take), context/sched.rs:1084-1176 (suspend with CPU stash) and
context/restore.rs (restore + replay). Page arithmetic follows runtime/src/api/inference.rs:914-942.
"""
from __future__ import annotations

import enum
import itertools
import threading
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

from ..driver.schema import CopyDir, CopyRequest
from .pagestore import PageStore, page_hash


class ContextError(RuntimeError):
    pass


class State(enum.Enum):
    ACTIVE = "active"
    PINNED = "pinned"
    SUSPENDED = "suspended"
    DESTROYED = "destroyed"


@dataclass
class Context:
    id: int
    model: str
    owner: str                        # process id ("" for snapshots)
    driver: int = 0
    chain: List[int] = field(default_factory=list)           # committed chain hashes
    working_pages: List[int] = field(default_factory=list)   # physical page ids
    tokens: List[int] = field(default_factory=list)          # lineage of the working area
    positions: List[int] = field(default_factory=list)
    mask_keys: List[bytes] = field(default_factory=list)     # per working token, b"" = causal
    committed_tokens: List[int] = field(default_factory=list)     # lineage of committed pages (for replay)
    committed_positions: List[int] = field(default_factory=list)
    max_committed_position: int = -1
    adapter_seed: int = 0
    state: State = State.ACTIVE
    pins: int = 0
    bid: float = 1.0
    stash: Optional[List[int]] = None    # host swap-pool page ids while suspended
    created_seq: int = 0

    @property
    def working_token_count(self) -> int:
        return len(self.tokens)


@dataclass
class PinnedContext:
    context_id: int
    pages: List[int]          # physical ids: committed then working
    kv_len: int               # committed_pages*page + working tokens
    driver: int
    rs_slot: int = -1         # recurrent-state slot (models with linear-attention layers), else -1
    rs_reset: int = 0         # 1: the next pass of this context starts its recurrent state from zero


class Deferred(ContextError):
    """The allocation must wait: pages are held back for, or can only come from, contexts that outrank the
    requester. `ContextManager.when_restorable` calls back when it is worth trying again."""


class ContextManager:
    """All contexts of one model. Thread-safe: inferlet host calls and the scheduler share it.

    Allocation order (`_alloc`; runtime/src/context/sched.rs:717-868): (1) priority gate - free pages
    that the head of the restore queue needs are not handed to a requester that does not outrank it;
    (2) the free pool; (3) the eviction loop, victims in market order; (4) defer - the requester's
    operation fails with `Deferred` and may queue itself with `when_restorable`."""

    def __init__(self, model: str, page_size: int, stores: Sequence[PageStore],
                 copy_fn: Optional[Callable[[int, CopyRequest], None]] = None,
                 swap_pages: int = 0, rs_slots: Sequence[int] = (),
                 rs_copy_fn: Optional[Callable[[int, int, int], None]] = None):
        self.model, self.page_size = model, page_size
        self.stores = list(stores)
        self.copy_fn = copy_fn or (lambda driver, req: None)
        self.contexts: Dict[int, Context] = {}
        self.snapshots: Dict[tuple, int] = {}      # (username, name) -> context id
        self.by_owner: Dict[str, set] = {}
        self._ids = itertools.count(1)
        self._seq = itertools.count(1)
        self.lock = threading.RLock()
        self._swap_free = list(range(swap_pages - 1, -1, -1))
        self.counters = {"created": 0, "forked": 0, "commits": 0, "dedup_pages": 0, "suspended": 0,
                         "restored": 0, "evictions": 0, "replayed_tokens": 0}
        self.market = None   # optional Market: orders eviction victims (defaulted, lowest bid, newest)
        self.media = None    # optional runtime.media.MediaRegistry: encoded clips held by the contexts' lineages
        # recurrent-state slot pools, one per driver (all empty for pure-attention models)
        from .rs_cache import RsCache
        self.rs = [RsCache(int(rs_slots[d]) if d < len(rs_slots) else 0) for d in range(len(self.stores))]
        self.rs_copy_fn = rs_copy_fn or (lambda driver, src, dst: None)
        self.restore_pause_at_utilization = 0.85
        self.restore_queue: Dict[int, list] = {d: [] for d in range(len(self.stores))}   # per driver: waiting contexts
        self.page_waiters: Dict[int, list] = {d: [] for d in range(len(self.stores))}    # one-shot callbacks
        self.counters.update({"deferred": 0, "gate_holds": 0, "restore_wakeups": 0})

    # ------------------------------------------------------------------ helpers
    def _get(self, cid: int) -> Context:
        ctx = self.contexts.get(cid)
        if ctx is None or ctx.state == State.DESTROYED:
            raise ContextError(f"context {cid} does not exist")
        return ctx

    def _store(self, ctx: Context) -> PageStore:
        return self.stores[ctx.driver]

    def _rank(self, ctx: Optional[Context]) -> tuple:
        """Higher outranks lower: (not defaulted, bid, older first)."""
        if ctx is None:
            return (0, float("-inf"), 0)
        defaulted = bool(self.market.defaulted(ctx.owner)) if self.market is not None else False
        return (0 if defaulted else 1, ctx.bid, -ctx.created_seq)

    def _restore_need(self, ctx: Context) -> int:
        """Pages a suspended context must be given to come back."""
        store = self._store(ctx)
        missing = len(ctx.chain) - store.prefix_len(ctx.chain)
        return missing + getattr(ctx, "_n_working", -(-len(ctx.tokens) // self.page_size))

    def _queue_head(self, driver: int) -> Optional[Context]:
        q = self.restore_queue[driver]
        while q:
            ctx = self.contexts.get(q[0][0])
            if ctx is not None and ctx.state == State.SUSPENDED:
                return ctx
            q.pop(0)                                   # restored by another path, or destroyed
        return None

    def _alloc(self, driver: int, n: int, exclude: Optional[int] = None) -> List[int]:
        store = self.stores[driver]
        requester = self.contexts.get(exclude) if exclude is not None else None
        head = self._queue_head(driver)
        if head is not None and head is not requester and self._rank(requester)[:2] < self._rank(head)[:2]:
            if store.pool.free_count - n < self._restore_need(head):
                self.counters["gate_holds"] += 1
                raise Deferred(f"KV pages are held for context {head.id}, which outranks the requester")
        pages = store.pool.alloc(n)
        while pages is None:
            if not self._evict_one(driver, exclude):
                self.counters["deferred"] += 1
                raise Deferred(f"out of KV pages: need {n}, free {store.pool.free_count}")
            pages = store.pool.alloc(n)
        return pages

    def least_loaded_driver(self) -> int:
        return max(range(len(self.stores)), key=lambda d: self.stores[d].pool.free_count)

    def best_driver_for(self, hashes: Sequence[int] = (), n_pages: int = 0) -> int:
        """Data-parallel placement: the replica where the context is cheapest to build - each page of the
        chain `hashes` already in a replica's store is a page that need not be computed or moved there;
        ties and empty chains go to the replica with the most free pages (sched.rs:367-417)."""
        with self.lock:
            def cost(d: int):
                present = self.stores[d].prefix_len(list(hashes)) if hashes else 0
                need = max(0, max(n_pages, len(hashes)) - present)
                short = max(0, need - self.stores[d].pool.free_count)      # pages that would need an eviction
                return (short, need, -self.stores[d].pool.free_count)
            return min(range(len(self.stores)), key=cost)

    # ------------------------------------------------------------------ restore admission
    def can_restore(self, cid: int) -> bool:
        """Whether a suspended context may come back now: its pages fit in what is free plus what contexts
        it outranks could give up, and - unless it heads the queue of an otherwise idle pool - the pool
        stays under `restore_pause_at_utilization` afterwards (sched.rs:881-938)."""
        with self.lock:
            ctx = self._get(cid)
            if ctx.state != State.SUSPENDED:
                return True
            store = self._store(ctx)
            need = self._restore_need(ctx)
            free = store.pool.free_count
            total = free + store.pool.used_count
            if need <= free:
                head = self._queue_head(ctx.driver)
                if head is None or head is ctx or self._rank(ctx)[:2] >= self._rank(head)[:2]:
                    return (total - free + need) <= self.restore_pause_at_utilization * total or \
                        not any(c.pins for c in self.contexts.values() if c.driver == ctx.driver)
                return free - need >= self._restore_need(head)
            mine = self._rank(ctx)
            evictable = sum(len(c.working_pages) + store.would_free(c.chain) for c in self.contexts.values()
                            if c.driver == ctx.driver and c.state == State.ACTIVE and c.pins == 0 and c is not ctx
                            and self._rank(c)[:2] <= mine[:2])
            return need <= free + evictable

    def when_restorable(self, cid: int, callback: Callable[[], None]) -> None:
        """Queue a suspended context (best rank first, then arrival); `callback` runs once, outside the
        lock, when pages were freed and `can_restore` holds - or at once if it already does."""
        with self.lock:
            ctx = self._get(cid)
            if ctx.state != State.SUSPENDED or self.can_restore(cid):
                ready = True
            else:
                ready = False
                q = self.restore_queue[ctx.driver]
                q.append((cid, callback, next(self._seq)))
                q.sort(key=lambda e: (tuple(-x for x in self._rank(self.contexts[e[0]])[:2]) if e[0] in self.contexts
                                      else (0, 0), e[2]))
        if ready:
            callback()

    def _waiting(self, driver: int) -> bool:
        return bool(self.restore_queue[driver] or self.page_waiters[driver])

    def on_pages_freed(self, driver: int, callback: Callable[[], None]) -> None:
        """One-shot: `callback` runs (outside the lock) the next time pages of `driver` are given back.
        For requesters that were deferred while resident (growth under contention)."""
        with self.lock:
            self.page_waiters[driver].append(callback)

    def _pages_freed(self, driver: int) -> None:
        """Wake the waiters that can come back now, best rank first, then the deferred growers. Call
        without the lock held."""
        ready = []
        with self.lock:
            q = self.restore_queue[driver]
            while q:
                cid, cb, _ = q[0]
                ctx = self.contexts.get(cid)
                if ctx is None or ctx.state != State.SUSPENDED:
                    q.pop(0)
                    if ctx is not None:
                        ready.append(cb)
                    continue
                if not self.can_restore(cid):
                    break
                q.pop(0)
                ready.append(cb)
            self.counters["restore_wakeups"] += len(ready)
            ready += self.page_waiters[driver]
            self.page_waiters[driver] = []
        for cb in ready:
            cb()

    # ------------------------------------------------------------------ lifecycle
    def create(self, owner: str, driver: Optional[int] = None) -> int:
        with self.lock:
            cid = next(self._ids)
            d = self.least_loaded_driver() if driver is None else driver
            self.contexts[cid] = Context(id=cid, model=self.model, owner=owner, driver=d,
                                         created_seq=next(self._seq))
            self.by_owner.setdefault(owner, set()).add(cid)
            self.counters["created"] += 1
            return cid

    def destroy(self, cid: int) -> None:
        with self.lock:
            ctx = self.contexts.get(cid)
            if ctx is None or ctx.state == State.DESTROYED:
                return
            store = self._store(ctx)
            store.release(ctx.chain)
            store.pool.free(ctx.working_pages)
            if ctx.stash:
                self._swap_free.extend(ctx.stash)
            ctx.chain, ctx.working_pages, ctx.stash = [], [], None
            self.rs[ctx.driver].forget(cid)
            if self.media is not None:
                self.media.drop(cid)
            ctx.state = State.DESTROYED
            self.by_owner.get(ctx.owner, set()).discard(cid)
            del self.contexts[cid]
            waiting = self._waiting(ctx.driver)
        if waiting:
            self._pages_freed(ctx.driver)

    def destroy_owner(self, owner: str) -> None:
        with self.lock:
            for cid in list(self.by_owner.get(owner, ())):
                self.destroy(cid)
            self.by_owner.pop(owner, None)

    # ------------------------------------------------------------------ queries
    # The three counters are read without the lock: each is one dictionary look-up and one list length,
    # which the interpreter reads atomically, and the only writer that moves pages between the two lists
    # (commit) runs on the context owner's own thread. An inferlet asks for them on every step; under
    # the lock each call could wait for a whole batch delivery on the scheduler thread.
    def committed_page_count(self, cid: int) -> int:
        return len(self._get(cid).chain)

    def working_page_count(self, cid: int) -> int:
        return len(self._get(cid).working_pages)

    def working_page_token_count(self, cid: int) -> int:
        return len(self._get(cid).tokens)

    def kv_len(self, cid: int) -> int:
        with self.lock:
            ctx = self._get(cid)
            return len(ctx.chain) * self.page_size + len(ctx.tokens)

    # ------------------------------------------------------------------ working pages
    def reserve_working_pages(self, cid: int, n: int) -> None:
        with self.lock:
            ctx = self._get(cid)
            self._ensure_resident(ctx)
            ctx.working_pages.extend(self._alloc(ctx.driver, n, exclude=cid))

    def release_working_pages(self, cid: int, n: int) -> None:
        with self.lock:
            ctx = self._get(cid)
            n = min(n, len(ctx.working_pages))
            keep = len(ctx.working_pages) - n
            if keep * self.page_size < len(ctx.tokens):
                # tokens living in released pages are dropped with them
                self._truncate_to(ctx, keep * self.page_size)
            freed, ctx.working_pages = ctx.working_pages[keep:], ctx.working_pages[:keep]
            self._store(ctx).pool.free(freed)
            waiting = self._waiting(ctx.driver)
        if waiting:
            self._pages_freed(ctx.driver)

    def truncate_working_page_tokens(self, cid: int, n: int) -> None:
        with self.lock:
            ctx = self._get(cid)
            self._truncate_to(ctx, max(0, len(ctx.tokens) - n))

    def _truncate_to(self, ctx: Context, keep: int) -> None:
        if keep < len(ctx.tokens):
            self.rs[ctx.driver].invalidate(ctx.id)     # a recurrent state cannot be rolled back: replay
        del ctx.tokens[keep:], ctx.positions[keep:], ctx.mask_keys[keep:]

    def append_working_tokens(self, cid: int, tokens: Sequence[int], positions: Sequence[int],
                              mask_keys: Optional[Sequence[bytes]] = None) -> None:
        """Record tokens whose KV a finished forward pass wrote at the tail of the context."""
        with self.lock:
            ctx = self._get(cid)
            if len(ctx.tokens) + len(tokens) > len(ctx.working_pages) * self.page_size:
                raise ContextError("KV_INVARIANT_VIOLATION: working tokens exceed working pages")
            if len(tokens) == 1 and mask_keys is None:           # a decode step: one token, no generator objects
                ctx.tokens.append(int(tokens[0]))
                ctx.positions.append(int(positions[0]))
                ctx.mask_keys.append(b"")
                return
            ctx.tokens.extend(int(t) for t in tokens)
            ctx.positions.extend(int(p) for p in positions)
            ctx.mask_keys.extend(mask_keys if mask_keys is not None else [b""] * len(tokens))

    def commit_working_pages(self, cid: int, n: int) -> None:
        """Turn the first n (full) working pages into committed, shareable pages."""
        with self.lock:
            ctx = self._get(cid)
            ps = self.page_size
            if n > len(ctx.working_pages) or n * ps > len(ctx.tokens):
                raise ContextError("commit needs full working pages")
            pos = ctx.positions[: n * ps]
            last = ctx.max_committed_position
            for p in pos:
                if p <= last:
                    raise ContextError("committed positions must be strictly increasing")
                last = p
            store = self._store(ctx)
            prev = ctx.chain[-1] if ctx.chain else 0
            for i in range(n):
                tok = ctx.tokens[i * ps:(i + 1) * ps]
                pp = ctx.positions[i * ps:(i + 1) * ps]
                mk = b"".join(ctx.mask_keys[i * ps:(i + 1) * ps])
                h = page_hash(prev, tok, pp, mk, ctx.adapter_seed)
                page, dedup = store.extend(prev, h, ctx.working_pages[i])
                if dedup:
                    store.pool.free([ctx.working_pages[i]])
                    self.counters["dedup_pages"] += 1
                ctx.chain.append(h)
                prev = h
            ctx.committed_tokens.extend(ctx.tokens[: n * ps])
            ctx.committed_positions.extend(pos)
            ctx.max_committed_position = last
            del ctx.working_pages[:n]
            self._truncate_front(ctx, n * ps)
            self.counters["commits"] += 1

    def _truncate_front(self, ctx: Context, n: int) -> None:
        del ctx.tokens[:n], ctx.positions[:n], ctx.mask_keys[:n]

    # ------------------------------------------------------------------ fork / snapshots
    def fork(self, cid: int, owner: Optional[str] = None) -> int:
        """Share the committed chain, physically copy the working pages."""
        with self.lock:
            src = self._get(cid)
            self._ensure_resident(src)
            store = self._store(src)
            new_pages = self._alloc(src.driver, len(src.working_pages), exclude=cid)
            store.acquire(src.chain)
            if new_pages:
                self.copy_fn(src.driver, CopyRequest(CopyDir.D2D, np.asarray(src.working_pages, np.int32),
                                                     np.asarray(new_pages, np.int32)))
            nid = next(self._ids)
            own = src.owner if owner is None else owner
            self.contexts[nid] = Context(
                id=nid, model=self.model, owner=own, driver=src.driver, chain=list(src.chain),
                working_pages=new_pages, tokens=list(src.tokens), positions=list(src.positions),
                mask_keys=list(src.mask_keys), committed_tokens=list(src.committed_tokens),
                committed_positions=list(src.committed_positions),
                max_committed_position=src.max_committed_position, adapter_seed=src.adapter_seed,
                bid=src.bid, created_seq=next(self._seq))
            self.by_owner.setdefault(own, set()).add(nid)
            self.counters["forked"] += 1
            if self.media is not None:
                self.media.fork(cid, nid)       # the child's lineage holds the parent's clips
            rs = self.rs[src.driver]
            if rs.supported:
                from .rs_cache import RsState
                pair = rs.fork(cid, nid) if not own.startswith("@snapshot") else None
                if pair is not None:
                    self.rs_copy_fn(src.driver, pair[0], pair[1])
                elif rs.state_of(cid) != RsState.EMPTY or own.startswith("@snapshot"):
                    rs.state[nid] = RsState.MISSING if (src.chain or src.tokens) else RsState.EMPTY
            return nid

    def save(self, cid: int, username: str, name: str) -> None:
        with self.lock:
            key = (username, name)
            if key in self.snapshots:
                self.destroy(self.snapshots.pop(key))
            snap = self.fork(cid, owner=f"@snapshot:{username}")
            self.snapshots[key] = snap

    def snapshot(self, cid: int, username: str) -> str:
        name = f"snap-{next(self._seq):08x}"
        self.save(cid, username, name)
        return name

    def open(self, username: str, name: str, owner: str) -> int:
        with self.lock:
            snap = self.snapshots.get((username, name))
            if snap is None:
                raise ContextError(f"no snapshot named {name!r}")
            return self.fork(snap, owner=owner)

    def take(self, username: str, name: str, owner: str) -> int:
        with self.lock:
            snap = self.snapshots.pop((username, name), None)
            if snap is None:
                raise ContextError(f"no snapshot named {name!r}")
            ctx = self._get(snap)
            self.by_owner.get(ctx.owner, set()).discard(snap)
            ctx.owner = owner
            self.by_owner.setdefault(owner, set()).add(snap)
            return snap

    def delete_snapshot(self, username: str, name: str) -> None:
        with self.lock:
            snap = self.snapshots.pop((username, name), None)
            if snap is None:
                raise ContextError(f"no snapshot named {name!r}")
            self.destroy(snap)

    # ------------------------------------------------------------------ pin / unpin
    def pin(self, cid: int, n_new_tokens: int) -> PinnedContext:
        """Freeze the page list for a forward pass that appends n_new_tokens at the tail."""
        with self.lock:
            ctx = self._get(cid)
            self._ensure_resident(ctx)
            ps = self.page_size
            kv_len = len(ctx.chain) * ps + len(ctx.tokens)
            cap = (len(ctx.chain) + len(ctx.working_pages)) * ps
            if kv_len + n_new_tokens > cap:
                raise ContextError(
                    f"KV_INVARIANT_VIOLATION: kv_len {kv_len} + {n_new_tokens} inputs > capacity {cap}")
            rs_slot, rs_reset = -1, 0
            rs = self.rs[ctx.driver]
            if rs.supported:
                from .rs_cache import RsState
                rs_slot = rs.acquire(cid)
                if rs_slot is None:
                    victim = self._rs_victim(ctx)
                    if victim is None:
                        self.counters["deferred"] += 1
                        raise Deferred("no free recurrent-state slot")
                    rs.release(victim.id)
                    rs_slot = rs.acquire(cid)
                if rs.state_of(cid) == RsState.MISSING and kv_len > 0 and not getattr(ctx, "_pending_replay", None):
                    # the state was lost (eviction, truncation, opened from a snapshot): rebuild it by running
                    # the whole lineage again, committed part included
                    spans = []
                    if ctx.committed_tokens:
                        spans.append((list(ctx.committed_tokens), list(ctx.committed_positions), 0))
                    if ctx.tokens:
                        spans.append((list(ctx.tokens), list(ctx.positions), len(ctx.chain) * ps))
                    ctx._pending_replay = spans
                    self.counters["replayed_tokens"] += sum(len(sp[0]) for sp in spans)
                rs_reset = 1 if rs.flags_for_pass(cid) else 0
            ctx.pins += 1
            ctx.state = State.PINNED
            # physical ids of the committed chain: looked up once per chain length (a resident chain's pages
            # do not move; suspend / restore drop the cache), not once per forward pass
            cached = ctx.__dict__.get("_phys")
            if cached is None or cached[0] != len(ctx.chain):
                cached = ctx.__dict__["_phys"] = (len(ctx.chain), self._store(ctx).physical_ids(ctx.chain))
            pages = cached[1] + ctx.working_pages
            return PinnedContext(cid, pages, kv_len, ctx.driver, rs_slot if rs_slot is not None else -1, rs_reset)

    def _rs_victim(self, requester: Context) -> Optional[Context]:
        """An unpinned context whose recurrent-state slot may be taken (lowest rank first)."""
        rs = self.rs[requester.driver]
        cands = [c for c in self.contexts.values() if c.driver == requester.driver and c.pins == 0
                 and c is not requester and c.id in rs.slot_of]
        return min(cands, key=self._rank) if cands else None

    def unpin(self, cid: int) -> None:
        with self.lock:
            ctx = self.contexts.get(cid)
            if ctx is None:
                return
            ctx.pins = max(0, ctx.pins - 1)
            if ctx.pins == 0 and ctx.state == State.PINNED:
                ctx.state = State.ACTIVE
            waiting = ctx.pins == 0 and self._waiting(ctx.driver)
        if waiting:
            self._pages_freed(ctx.driver)       # an unpinned context is evictable again

    def pinned_count(self) -> int:
        with self.lock:
            return sum(1 for c in self.contexts.values() if c.pins > 0)

    def set_bid(self, cid: int, value: float) -> None:
        with self.lock:
            self._get(cid).bid = float(value)

    # ------------------------------------------------------------------ suspend / restore
    def suspend(self, cid: int) -> None:
        """Evict a context: stash working pages on the CPU tier when there is room (all or
        nothing), else drop them and remember the lineage for replay; release the chain."""
        with self.lock:
            ctx = self._get(cid)
            if ctx.state == State.SUSPENDED:
                return
            if ctx.pins:
                raise ContextError("cannot suspend a pinned context")
            store = self._store(ctx)
            used_working = -(-len(ctx.tokens) // self.page_size)
            stash = None
            if used_working and len(self._swap_free) >= used_working:
                stash = [self._swap_free.pop() for _ in range(used_working)]
                self.copy_fn(ctx.driver, CopyRequest(CopyDir.D2H, np.asarray(ctx.working_pages[:used_working], np.int32),
                                                     np.asarray(stash, np.int32)))
            ctx.stash = stash
            ctx._n_working = len(ctx.working_pages)
            store.pool.free(ctx.working_pages)
            ctx.working_pages = []
            ctx._chain_resident = store.would_free(ctx.chain) == 0
            store.release(ctx.chain)
            ctx.state = State.SUSPENDED
            ctx.__dict__.pop("_phys", None)
            self.rs[ctx.driver].release(cid)
            self.counters["suspended"] += 1

    def _ensure_resident(self, ctx: Context) -> None:
        if ctx.state == State.SUSPENDED:
            self.restore(ctx.id)

    def restore(self, cid: int) -> List[tuple]:
        """Bring a suspended context back. Returns the (tokens, positions, first_kv_index) spans
        that must be replayed through forward passes because their KV no longer exists."""
        with self.lock:
            ctx = self._get(cid)
            if ctx.state != State.SUSPENDED:
                return []
            if not self.can_restore(cid):
                self.counters["deferred"] += 1
                raise Deferred(f"context {cid} cannot be restored yet: {self._restore_need(ctx)} pages needed")
            store = self._store(ctx)
            ps = self.page_size
            # committed prefix still present in the store can simply be re-acquired
            present = store.prefix_len(ctx.chain)
            replay: List[tuple] = []
            if present < len(ctx.chain):
                missing = len(ctx.chain) - present
                pages = self._alloc(ctx.driver, missing, exclude=cid)
                store.acquire(ctx.chain[:present])
                prev = ctx.chain[present - 1] if present else 0
                for i, h in enumerate(ctx.chain[present:]):
                    store.extend(prev, h, pages[i])
                    prev = h
                a, b = present * ps, len(ctx.chain) * ps
                replay.append((ctx.committed_tokens[a:b], ctx.committed_positions[a:b], a))
                self.counters["replayed_tokens"] += b - a
            else:
                store.acquire(ctx.chain)
            n_working = getattr(ctx, "_n_working", -(-len(ctx.tokens) // ps))
            ctx.working_pages = self._alloc(ctx.driver, n_working, exclude=cid)
            if ctx.stash:
                self.copy_fn(ctx.driver, CopyRequest(CopyDir.H2D, np.asarray(ctx.stash, np.int32),
                                                     np.asarray(ctx.working_pages[:len(ctx.stash)], np.int32)))
                self._swap_free.extend(ctx.stash)
                ctx.stash = None
            elif ctx.tokens:
                replay.append((list(ctx.tokens), list(ctx.positions), len(ctx.chain) * ps))
                self.counters["replayed_tokens"] += len(ctx.tokens)
            ctx.state = State.ACTIVE
            self.counters["restored"] += 1
            if self.rs[ctx.driver].supported and (ctx.committed_tokens or ctx.tokens):
                # the recurrent state went with the slot: the next pin plans a replay of the whole lineage
                replay = []
            ctx._pending_replay = replay
            return replay

    def take_pending_replay(self, cid: int) -> List[tuple]:
        with self.lock:
            ctx = self._get(cid)
            r = getattr(ctx, "_pending_replay", [])
            ctx._pending_replay = []
            return r

    def _evict_one(self, driver: int, exclude: Optional[int]) -> bool:
        """Pick a victim (lowest bid, newest first) among unpinned resident contexts of the driver."""
        cands = [c for c in self.contexts.values()
                 if c.driver == driver and c.state == State.ACTIVE and c.pins == 0 and c.id != exclude
                 and (c.working_pages or c.chain) and not c.owner.startswith("@snapshot")]
        if not cands:
            cands = [c for c in self.contexts.values()
                     if c.driver == driver and c.state == State.ACTIVE and c.pins == 0 and c.id != exclude
                     and (c.working_pages or c.chain)]
        if not cands:
            return False
        if self.market is not None:
            victim = min(cands, key=lambda c: self.market.victim_key(c.owner, c.bid, c.created_seq))
        else:
            victim = min(cands, key=lambda c: (c.bid, -c.created_seq))
        requester = self.contexts.get(exclude) if exclude is not None else None
        if requester is not None and self._rank(victim)[:2] > self._rank(requester)[:2]:
            return False                 # the cheapest victim outranks the requester: the requester waits
        before = self.stores[driver].pool.free_count
        self.suspend(victim.id)
        self.counters["evictions"] += 1
        return self.stores[driver].pool.free_count > before

    # ------------------------------------------------------------------ accounting
    def pages_used(self, driver: int = 0) -> int:
        return self.stores[driver].pool.used_count

    def effective_pages(self, cid: int) -> float:
        with self.lock:
            ctx = self._get(cid)
            return self._store(ctx).effective_pages(ctx.chain, len(ctx.working_pages))

    def audit(self) -> None:
        """Every physical page is free, a working page of exactly one context, or a store node."""
        with self.lock:
            for d, store in enumerate(self.stores):
                owned = [p for c in self.contexts.values() if c.driver == d for p in c.working_pages]
                nodes = list(store.node_pages())
                if len(set(owned)) != len(owned):
                    raise ContextError("a working page is owned twice")
                if set(owned) & set(nodes):
                    raise ContextError("a page is both working and committed")
                if len(owned) + len(set(nodes)) != store.pool.used_count:
                    raise ContextError(
                        f"page leak: {len(owned)} working + {len(set(nodes))} committed != {store.pool.used_count} used")
