"""Batch scheduler: coalesces forward-pass calls of many inferlets into one ragged batch.

One OS thread per driver drains a queue of pending requests, accumulates them under the
driver's advertised limits, asks a policy whether to fire or wait, folds the per-request
arrays into one CSR `ForwardRequest`, runs it synchronously on the driver and scatters the
per-slot outputs back to the waiting futures. A request larger than `max_forward_tokens` is
split into sequential prefix chunks (chunked prefill).

Behavioural counterpart of runtime/src/inference/scheduler.rs:311-655 (accumulator and its
eight limits), :1173-1531 (run loop), :1545-1882 (execute_batch and scatter),
inference/adaptive_policy.rs:30-274 (policies), inference/scheduler/chunked.rs:48-293
(chunking) and inference/request.rs:387-540 (fold).
"""
from __future__ import annotations

import contextlib
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import numpy as np

from . import brle, telemetry
from ..driver.schema import Capabilities, ForwardRequest, ForwardResponse, SamplerSpec, SlotOutput, split_media_spans


class SlotList(list):
    """The slot outputs of one request, with the driver's verdict on its drafts when it gave one."""
    spec_accepted: Optional[int] = None


@dataclass
class PendingRequest:
    context_id: int
    tokens: Sequence[int]
    positions: Sequence[int]
    pages: Sequence[int]                  # physical pages: active prefix covering kv_len + len(tokens)
    kv_len: int                           # tokens already in the context
    samplers: List[tuple] = field(default_factory=list)   # (index within this request's tokens, SamplerSpec)
    masks: Optional[list] = None          # per input token BRLE over kv positions, None = causal
    logit_mask: Optional[list] = None     # BRLE over the vocabulary
    spec_count: int = 0                   # trailing input tokens that are unverified drafts
    adapter: int = -1
    rs_slot: int = -1                     # recurrent-state slot of the context (models with linear layers)
    rs_reset: int = 0                     # 1: the slot starts from zero in this pass
    on_done: Optional[Callable] = None    # called with (list[SlotOutput] | Exception)
    t_submit: float = 0.0
    chunk_of: Optional["_ChunkState"] = None

    @property
    def n_tokens(self) -> int:
        return len(self.tokens)


@dataclass
class _ChunkState:
    parent: PendingRequest
    offset: int = 0
    outputs: dict = field(default_factory=dict)   # original slot index -> SlotOutput
    reach: Optional[np.ndarray] = None            # with custom masks: running maximum of the last key each row may see


def mask_reach(masks: Sequence, kv_len: int) -> np.ndarray:
    """reach[i] = the largest key position that any of rows 0..i of the pass may attend (BRLE rows: even runs are
    zeros), never less than the row's own position. A row that looks past itself (bidirectional spans: image rows in
    Gemma-3, tree drafts) needs those keys written by the same fire, so a chunk may end after row i only if
    reach[i] <= kv_len + i."""
    out = np.empty(len(masks), dtype=np.int64)
    best = -1
    for i, runs in enumerate(masks):
        last, pos = kv_len + i, 0
        if runs is not None:
            for j, n in enumerate(runs):
                pos += n
                if j & 1 and n:
                    last = max(last, pos - 1)
        best = max(best, last)
        out[i] = best
    return out


@dataclass
class Usage:
    requests: int = 0
    tokens: int = 0
    page_refs: int = 0
    sampler_rows: int = 0
    mask_bytes: int = 0
    logprob_labels: int = 0
    logit_rows: int = 0        # distinct token rows that need the vocabulary projection
    prob_rows: int = 0         # distinct token rows that need a normalised distribution


_PROB_VALUES = None


def _needs_probs(spec) -> bool:
    global _PROB_VALUES
    if _PROB_VALUES is None:
        from ..driver.schema import SamplerKind
        _PROB_VALUES = frozenset(int(k) for k in (SamplerKind.DIST, SamplerKind.LOGPROB, SamplerKind.LOGPROBS,
                                                  SamplerKind.ENTROPY))
    return spec.kind.value in _PROB_VALUES          # plain ints: hashing an enum member runs Python code


class BatchAccumulator:
    """Admits requests while every one of the driver's eight limits holds: requests, tokens, page
    references, logit rows, probability rows, sampler rows, log-probability labels, custom-mask bytes
    (runtime/src/inference/scheduler.rs:311-655). Logit and probability rows are counted after the
    compact projection: samplers that read the same token row share one row."""

    def __init__(self, caps: Capabilities, page_size: int):
        self.caps, self.page_size = caps, page_size
        self.items: List[PendingRequest] = []
        self.usage = Usage()

    def cost(self, r: PendingRequest) -> Usage:
        total = r.kv_len + r.n_tokens
        pages = -(-total // self.page_size)
        mask_bytes = 0
        if r.masks is not None:
            mask_bytes = r.n_tokens * (-(-total // 8))
        if len(r.samplers) == 1:                     # the common case: one sampler on one row
            sp = r.samplers[0][1]
            labels, logit_rows, prob_rows = len(sp.labels), 1, 1 if _needs_probs(sp) else 0
        else:
            labels = sum(len(s.labels) for _, s in r.samplers)
            logit_rows = len({i for i, _ in r.samplers})
            prob_rows = len({i for i, s in r.samplers if _needs_probs(s)})
        return Usage(1, r.n_tokens, pages, len(r.samplers), mask_bytes, labels, logit_rows, prob_rows)

    def _cost(self, r: PendingRequest) -> Usage:
        c = r.__dict__.get("_usage")          # a request is costed by `fits` and again by `push`
        if c is None:
            c = r.__dict__["_usage"] = self.cost(r)
        return c

    def fits(self, r: PendingRequest) -> bool:
        c, u, caps = self._cost(r), self.usage, self.caps
        return (u.requests + c.requests <= caps.max_forward_requests
                and u.tokens + c.tokens <= caps.max_forward_tokens
                and u.page_refs + c.page_refs <= caps.max_page_refs
                and u.sampler_rows + c.sampler_rows <= caps.max_sampler_rows
                and u.logit_rows + c.logit_rows <= caps.max_logit_rows
                and u.prob_rows + c.prob_rows <= caps.max_prob_rows
                and u.mask_bytes + c.mask_bytes <= caps.max_custom_mask_bytes
                and u.logprob_labels + c.logprob_labels <= caps.max_logprob_labels)

    def push(self, r: PendingRequest) -> None:
        c, u = self._cost(r), self.usage
        u.requests += c.requests; u.tokens += c.tokens; u.page_refs += c.page_refs
        u.sampler_rows += c.sampler_rows; u.mask_bytes += c.mask_bytes; u.logprob_labels += c.logprob_labels
        u.logit_rows += c.logit_rows; u.prob_rows += c.prob_rows
        self.items.append(r)

    def take(self) -> List[PendingRequest]:
        items, self.items, self.usage = self.items, [], Usage()
        return items

    def __len__(self):
        return len(self.items)


def trim_plan(it: PendingRequest, page_size: int):
    """Page trim: pages whose KV positions are masked out in every row of the request's attention
    mask need not travel to the driver. Only pages before the first page that this pass writes
    qualify. Returns (kept page ids, re-indexed mask rows, number of dropped pages).
    Counterpart of runtime/src/inference/request.rs:109-229 (TrimPlan)."""
    first_writable = it.kv_len // page_size
    if it.masks is None or first_writable == 0:
        return None
    drop = brle.droppable_pages(it.masks, page_size, first_writable)
    nd = int(drop.sum())
    if nd == 0:
        return None
    pages = [p for i, p in enumerate(it.pages) if i >= first_writable or not drop[i]]
    masks = [brle.remove_pages(m, drop, page_size) for m in it.masks]
    return pages, masks, nd


def fold(items: Sequence[PendingRequest], page_size: int, trim: bool = True) -> ForwardRequest:
    """Per-request arrays -> one batched CSR request (page trim applied, decode masks elided)."""
    r = len(items)
    qo = np.zeros(r + 1, dtype=np.int32)
    pptr = np.zeros(r + 1, dtype=np.int32)
    last = np.zeros(r, dtype=np.int32)
    has_mask = np.zeros(r, dtype=bool)
    mask_ptr = np.zeros(r + 1, dtype=np.int32)
    tokens, positions, pages, mask_runs = [], [], [], []
    slot_req, slot_row, samplers = [], [], []
    logit_masks = [None] * r
    spec = np.zeros(r, dtype=np.int32)
    ctx_ids = np.zeros(r, dtype=np.uint64)
    adapters = np.full(r, -1, dtype=np.int64)
    rs_slots = np.full(r, -1, dtype=np.int32)
    rs_reset = np.zeros(r, dtype=np.int32)
    single = True
    trimmed = 0
    for i, it in enumerate(items):
        n = it.n_tokens
        single &= n == 1
        total = it.kv_len + n
        npg = -(-total // page_size)
        if npg > len(it.pages):
            raise ValueError("KV_INVARIANT_VIOLATION: request carries too few pages")
        it_pages, it_masks = it.pages, it.masks
        plan = trim_plan(it, page_size) if trim and it.masks is not None else None
        if plan is not None:
            it_pages, it_masks, nd = plan
            trimmed += nd
            npg -= nd
            total -= nd * page_size
        tokens.append(np.asarray(it.tokens, dtype=np.int32))
        positions.append(np.asarray(it.positions, dtype=np.int32))
        pages.append(np.asarray(it_pages[:npg], dtype=np.int32))
        qo[i + 1] = qo[i] + n
        pptr[i + 1] = pptr[i] + npg
        last[i] = total % page_size or (page_size if total else 0)
        if it_masks is not None:
            has_mask[i] = True
            mask_runs.extend(it_masks)
        mask_ptr[i + 1] = len(mask_runs)
        for idx, sp in it.samplers:
            slot_req.append(i)
            slot_row.append(int(qo[i]) + idx)
            samplers.append(sp)
        logit_masks[i] = it.logit_mask
        spec[i] = it.spec_count
        ctx_ids[i] = it.context_id
        adapters[i] = it.adapter
        rs_slots[i], rs_reset[i] = it.rs_slot, it.rs_reset
    cat = lambda xs: np.concatenate(xs) if xs else np.zeros(0, dtype=np.int32)
    any_mask = bool(has_mask.any())
    # media placeholders in the lineage become spans of the side channel; the driver sees token 0 there
    toks, m_slot, m_src, m_dst, m_cnt = split_media_spans(cat(tokens))
    return ForwardRequest(
        tokens=toks, positions=cat(positions), qo_indptr=qo, kv_page_indices=cat(pages),
        media_slot=m_slot, media_src=m_src, media_dst=m_dst, media_count=m_cnt,
        kv_page_indptr=pptr, kv_last_page_lens=last,
        has_user_mask=has_mask if any_mask else None, mask_runs=mask_runs if any_mask else None,
        mask_row_indptr=mask_ptr if any_mask else None,
        logit_masks=logit_masks if any(m is not None for m in logit_masks) else None,
        slot_req=np.asarray(slot_req, dtype=np.int32), slot_row=np.asarray(slot_row, dtype=np.int32),
        slot_samplers=samplers, spec_counts=spec if spec.any() else None, context_ids=ctx_ids,
        adapter_ids=adapters, single_token_mode=single, trimmed_pages=trimmed,
        rs_slots=rs_slots if (rs_slots >= 0).any() else None, rs_reset=rs_reset if (rs_slots >= 0).any() else None)


# ------------------------------------------------------------------------------ policies
class Policy:
    def decide(self, batch_size: int, waited_s: float, sched: "BatchScheduler") -> float:
        """Return 0 to fire now, or the number of seconds to keep waiting for more requests."""
        raise NotImplementedError

    def after_fire(self, batch_size: int, latency_s: float) -> None:
        pass


class GreedyPolicy(Policy):
    def decide(self, batch_size, waited_s, sched):
        return 0.0


class EagerPolicy(Policy):
    """Fire when every context that is currently pinned-or-pending has joined the batch."""

    def __init__(self, max_wait_s: float = 0.002):
        self.max_wait_s = max_wait_s

    def decide(self, batch_size, waited_s, sched):
        cohort = sched.cohort_size()
        if batch_size >= cohort or waited_s >= self.max_wait_s:
            return 0.0
        return self.max_wait_s - waited_s


class AdaptivePolicy(Policy):
    """Fire at the driver cap, at the recent cohort high-water mark, or when the wait reaches the
    last batch latency (watchdog). The high-water mark relaxes by one per fire so that a
    shrinking population of inferlets does not stall on a stale target."""

    def __init__(self, min_wait_s: float = 0.0002, max_wait_s: float = 0.050):
        self.high_water = 1
        self.last_latency = 0.001
        self.min_wait_s, self.max_wait_s = min_wait_s, max_wait_s

    def decide(self, batch_size, waited_s, sched):
        if batch_size >= sched.caps.max_forward_requests or batch_size >= self.high_water:
            return 0.0
        budget = min(self.max_wait_s, max(self.min_wait_s, self.last_latency))
        if waited_s >= budget:
            return 0.0
        return budget - waited_s

    def after_fire(self, batch_size, latency_s):
        self.last_latency = latency_s
        self.high_water = max(batch_size, self.high_water - 1, 1)


def make_policy(name: str) -> Policy:
    return {"adaptive": AdaptivePolicy, "eager": EagerPolicy, "greedy": GreedyPolicy}[name]()


# ------------------------------------------------------------------------------ scheduler
class BatchScheduler:
    def __init__(self, driver, caps: Capabilities, page_size: int, policy: str = "adaptive",
                 on_batch: Optional[Callable] = None, name: str = "pie-sched-0"):
        self.driver, self.caps, self.page_size = driver, caps, page_size
        self.policy = make_policy(policy)
        self.q: "queue.SimpleQueue[Optional[PendingRequest]]" = queue.SimpleQueue()
        self.acc = BatchAccumulator(caps, page_size)
        self.stash: Optional[PendingRequest] = None
        self._last_fire_start = 0.0
        self._last_dispatch_end = 0.0
        self.on_batch = on_batch
        self.post_fire_hooks: List[Callable] = []
        # Held (re-entrantly) while the results of one fire are scattered to their requests: every
        # delivery takes the context manager's lock a few times, and taking it once around the whole
        # loop keeps the inferlet thread from interleaving with each of several hundred deliveries.
        self.delivery_guard = contextlib.nullcontext()
        self.running = True
        self.aborted: Optional[Exception] = None
        self.inflight_contexts = 0
        self.stats = {"total_batches": 0, "total_requests": 0, "total_tokens": 0, "last_latency_us": 0.0,
                      "cum_latency_us": 0.0, "batch_size_hist": [0] * 8, "chunked_requests": 0,
                      "failed_batches": 0}
        self.expected_cohort: Callable[[], int] = lambda: 0
        self.cohort = None            # DecodeCohort of this driver (set by the engine)
        self._inflight = None         # (AsyncTokens, row snapshot) of the pipelined decode step
        self._parity = 0
        self.thread = threading.Thread(target=self.run, name=name, daemon=True)
        self.thread.start()

    # ---- producer side
    def submit(self, r: PendingRequest) -> None:
        if self.aborted is not None:
            if r.on_done:
                r.on_done(self.aborted)
            return
        r.t_submit = time.perf_counter()
        self.q.put(r)

    def cohort_size(self) -> int:
        return max(1, self.expected_cohort())

    def abort(self, exc: Exception) -> None:
        """Fail everything in flight and everything submitted from now on (driver death)."""
        self.aborted = exc
        self.running = False
        self.q.put(None)

    def shutdown(self) -> None:
        self.running = False
        self.q.put(None)
        self.thread.join(timeout=5)

    # ---- chunked prefill
    MIN_HEAD_CHUNK = 64      # a partially filled batch takes the head of a long prefill only if this many tokens fit

    def _prepare(self, r: PendingRequest) -> PendingRequest:
        """A request longer than the driver's token limit becomes a chain of prefix chunks
        (runtime/src/inference/scheduler/chunked.rs:48-293): each chunk is an ordinary request over
        the same page list with `kv_len` advanced, samplers and masks sliced to its rows; the parent is
        answered once, in attach order, after the last chunk - or with the first failure."""
        cap = self.caps.max_forward_tokens
        if r.n_tokens <= cap or r.chunk_of is not None:
            return r
        self.stats["chunked_requests"] += 1
        st = _ChunkState(parent=r)
        return self._next_chunk(st)

    def _next_chunk(self, st: _ChunkState, limit: Optional[int] = None) -> PendingRequest:
        p = st.parent
        cap = min(self.caps.max_forward_tokens, limit or self.caps.max_forward_tokens)
        a, b = st.offset, min(st.offset + cap, p.n_tokens)
        if b < p.n_tokens:
            # end an inner chunk on a page boundary when that still makes progress: the next chunk then
            # starts a fresh page and no page is written by two fires
            aligned = b - (p.kv_len + b) % self.page_size
            if aligned > a:
                b = aligned
            # and never past what the sampler-row limits admit in one fire
            rows = sorted({idx for idx, _ in p.samplers if a <= idx < b})
            lim = min(self.caps.max_logit_rows, self.caps.max_sampler_rows)
            if len(rows) > lim:
                b = rows[lim]
            if p.masks is not None:
                # rows that look ahead of themselves keep the keys they look at in their own fire
                if st.reach is None:
                    st.reach = mask_reach(p.masks, p.kv_len)
                c = b
                while c > a and st.reach[c - 1] > p.kv_len + c - 1:
                    c -= 1
                if c == a:          # no cut point inside the budget: take the whole look-ahead span, or fail on the limits
                    c = b
                    while c < p.n_tokens and st.reach[c - 1] > p.kv_len + c - 1:
                        c += 1
                b = c
        samplers = [(idx - a, sp) for idx, sp in p.samplers if a <= idx < b]
        st._slot_ids = [k for k, (idx, _) in enumerate(p.samplers) if a <= idx < b]
        # drafts of a chunked request are verified by the runtime from the slots, not per chunk
        return PendingRequest(
            context_id=p.context_id, tokens=p.tokens[a:b], positions=p.positions[a:b], pages=p.pages,
            kv_len=p.kv_len + a, samplers=samplers, masks=None if p.masks is None else p.masks[a:b],
            logit_mask=p.logit_mask, adapter=p.adapter, chunk_of=st, t_submit=p.t_submit,
            rs_slot=p.rs_slot, rs_reset=p.rs_reset if a == 0 else 0)

    # ---- consumer side
    def _admit(self, r: PendingRequest) -> bool:
        r = self._prepare(r)
        if self.acc.fits(r):
            self.acc.push(r)
            return True
        if len(self.acc) == 0:
            if r.on_done or r.chunk_of:
                self._deliver(r, ValueError("request exceeds the driver's forward limits"))
            return True
        # a long prefill behind a partially filled batch: its head rides along in the tokens that are left
        room = self.caps.max_forward_tokens - self.acc.usage.tokens
        if room >= self.MIN_HEAD_CHUNK and r.n_tokens > room and (r.chunk_of is None or r.chunk_of.offset + r.n_tokens
                                                                  <= r.chunk_of.parent.n_tokens):
            st = r.chunk_of
            if st is None:
                st = _ChunkState(parent=r)
                self.stats["chunked_requests"] += 1
            head = self._next_chunk(st, limit=room)
            if head.n_tokens < r.n_tokens and self.acc.fits(head):
                self.stats["head_chunks"] = self.stats.get("head_chunks", 0) + 1
                self.acc.push(head)
                return True
            if r.chunk_of is None:
                self.stats["chunked_requests"] -= 1
        self.stash = r
        return False

    def _cohort_busy(self) -> bool:
        return self._inflight is not None or (self.cohort is not None and self.cohort.has_work())

    def _drain_inflight(self) -> None:
        if self._inflight is not None:
            handle, snap = self._inflight
            self._inflight = None
            self.cohort.absorb(snap, handle.wait())

    def _cohort_step(self) -> None:
        """Launch decode step s, then absorb step s-1 while s runs on the GPU."""
        t0 = time.perf_counter()
        built = self.cohort.build() if self.cohort.has_work() else None
        handle = None
        if built is not None:
            step, snap = built
            handle = self.driver.decode_async(step, self._parity)
            self._parity ^= 1
        self._drain_inflight()
        if handle is not None:
            self._inflight = (handle, snap)
            st = self.stats
            st["total_batches"] += 1
            st["total_requests"] += step.r
            st["total_tokens"] += step.r
            st["decode_steps"] = st.get("decode_steps", 0) + 1
            lat = time.perf_counter() - t0
            st["last_latency_us"] = lat * 1e6
            st["cum_latency_us"] += lat * 1e6
            st["batch_size_hist"][min(7, max(1, step.r).bit_length() - 1)] += 1
            if self.post_fire_hooks and (st["decode_steps"] & 15) == 0:   # market tick every 16 decode steps
                ids = [s_.ctx_id for s_ in snap]
                for hook in self.post_fire_hooks:
                    hook(ids)
            if self.on_batch:
                self.on_batch(step.r, step.r, lat, "decode")

    def run(self) -> None:
        while self.running:
            try:
                busy = self._cohort_busy()
                if self.stash is not None:
                    r, self.stash = self.stash, None
                elif busy:
                    try:
                        r = self.q.get_nowait()
                    except queue.Empty:
                        r = None
                else:
                    r = self.q.get()
                if r is not None:
                    # an ordinary batch shares the input slab: finish the pipelined step first
                    self._drain_inflight()
                    t_first = time.perf_counter()
                    self._admit(r)
                    while self.stash is None:
                        try:
                            while self.stash is None:
                                nxt = self.q.get_nowait()
                                if nxt is None:
                                    break
                                self._admit(nxt)
                        except queue.Empty:
                            pass
                        if self.stash is not None or not self.running or busy:
                            break
                        wait = self.policy.decide(len(self.acc), time.perf_counter() - t_first, self)
                        if wait <= 0:
                            break
                        try:
                            nxt = self.q.get(timeout=wait)
                            if nxt is not None:
                                self._admit(nxt)
                        except queue.Empty:
                            break
                    if len(self.acc):
                        self.execute_batch(self.acc.take(), time.perf_counter() - t_first)
                if self.cohort is not None and self._cohort_busy():
                    self._cohort_step()
            except Exception as e:  # keep the scheduler alive; fail what was in flight
                for it in self.acc.take():
                    self._deliver(it, e)
                if self.cohort is not None:
                    self._inflight = None
                    self.cohort.abort_all(e)
        exc = self.aborted or RuntimeError("scheduler stopped")
        for it in self.acc.take():
            self._deliver(it, exc)
        if self.cohort is not None:
            self._inflight = None
            self.cohort.abort_all(exc)
        while True:
            try:
                it = self.q.get_nowait()
            except queue.Empty:
                break
            if it is not None:
                self._deliver(it, exc)

    def execute_batch(self, items: List[PendingRequest], t_accum: float = 0.0) -> None:
        """One fire. With telemetry on, records the per-fire probe tree (runtime/src/probe/fire.rs:9-30):
        fire_inter_fire / fire_post_dispatch_to_fire (gaps between fires, siblings of the rest),
        fire_accumulate_loop, fire_execute_{batch_build, driver_fire, response_dispatch, total} (the three
        children sum to the total), fire_post_dispatch_hooks, and the driver's own split of its fire
        (driver_{build, h2d, forward, sample, d2h, total}; runtime/src/probe/driver_cuda.rs)."""
        t0 = time.perf_counter()
        tel = telemetry.get()
        try:
            req = fold(items, self.page_size)
            t_built = time.perf_counter()
            resp: ForwardResponse = self.driver.fire_batch(req)
        except Exception as e:
            self.stats["failed_batches"] += 1
            for it in items:
                self._deliver(it, e)
            return
        t_fired = time.perf_counter()
        lat = t_fired - t0
        if tel.enabled:
            tel.incr("fires")
            tel.incr("forward_tokens", req.num_tokens)
            us = tel.record_probe_us
            us("fire_batch", lat * 1e6)
            if self._last_fire_start:
                us("fire_inter_fire", (t0 - self._last_fire_start) * 1e6)
                us("fire_post_dispatch_to_fire", (t0 - self._last_dispatch_end) * 1e6)
            self._last_fire_start = t0
            us("fire_accumulate_loop", t_accum * 1e6)
            us("fire_execute_batch_build", (t_built - t0) * 1e6)
            us("fire_execute_driver_fire", (t_fired - t_built) * 1e6)
            for k in ("build", "h2d", "forward", "sample", "d2h", "total"):
                us(f"driver_{k}", getattr(resp, f"t_{k}_us", 0.0))
        st = self.stats
        st["total_batches"] += 1
        st["total_requests"] += len(items)
        st["total_tokens"] += req.num_tokens
        st["trimmed_pages"] = st.get("trimmed_pages", 0) + req.trimmed_pages
        st["last_latency_us"] = lat * 1e6
        st["cum_latency_us"] += lat * 1e6
        st["batch_size_hist"][min(7, max(0, len(items)).bit_length() - 1 if len(items) else 0)] += 1
        self.policy.after_fire(len(items), lat)
        if len(resp.slots) != len(req.slot_samplers):
            err = RuntimeError(f"driver returned {len(resp.slots)} slots for {len(req.slot_samplers)} samplers")
            for it in items:
                self._deliver(it, err)
            return
        k = 0
        with self.delivery_guard:
            for ri, it in enumerate(items):
                n = len(it.samplers)
                out = SlotList(resp.slots[k:k + n])
                if resp.spec_accepted is not None:
                    out.spec_accepted = int(resp.spec_accepted[ri])
                self._deliver(it, out)
                k += n
            t_disp = time.perf_counter()
            for hook in self.post_fire_hooks:
                hook([it.context_id for it in items])
        if self.on_batch:
            self.on_batch(len(items), req.num_tokens, lat, "batch")
        if tel.enabled:
            self._last_dispatch_end = time.perf_counter()
            tel.record_probe_us("fire_execute_response_dispatch", (t_disp - t_fired) * 1e6)
            tel.record_probe_us("fire_execute_total", (t_disp - t0) * 1e6)
            tel.record_probe_us("fire_post_dispatch_hooks", (self._last_dispatch_end - t_disp) * 1e6)

    def _deliver(self, it: PendingRequest, result) -> None:
        st = it.chunk_of
        if st is not None:
            p = st.parent
            if isinstance(result, Exception):
                if p.on_done:
                    p.on_done(result)
                return
            for sid, out in zip(st._slot_ids, result):
                st.outputs[sid] = out
            st.offset += it.n_tokens
            if st.offset < p.n_tokens:
                nxt = self._next_chunk(st)
                nxt.t_submit = time.perf_counter()
                self.q.put(nxt)
                return
            if p.on_done:
                p.on_done([st.outputs[i] for i in range(len(p.samplers))])
            return
        if it.on_done:
            it.on_done(result)
