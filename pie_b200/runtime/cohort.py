"""Decode cohort: the array-form hot loop for plain token generation.

A *stream* is a context in steady decode (one sampled token per step, fed back as the next
input) with a plain token sampler, a token budget and a stop set. All streams of a driver
live in one set of numpy arrays (row = stream): positions, KV lengths, page tables, sampler
parameters and a token buffer, so that building the next batch and absorbing its results is
a handful of vectorised operations instead of per-request object traffic.

The scheduler pipelines the cohort one step deep: step s is launched (its input tokens are
fed on the device from step s-1's samples) BEFORE the host has looked at step s-1's tokens;
stop conditions are therefore detected one step late and a finished stream simply rides along
for one extra, discarded step. This is the pass-level speculation of the reference
(runtime/src/inference/speculator.rs:1-24: the next single-token pass is built from the
sampled token and submitted before the inferlet asks for it) taken to its limit: the
speculated pass is built on the device, not on the host.

Context bookkeeping (lineage append, page commits) is done in bulk when a stream ends or the
inferlet touches the context again, not per token.
"""
from __future__ import annotations

import itertools
import threading
import time
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

from ..driver.executor import CohortStep
from ..driver.schema import SamplerKind, SamplerSpec, position_seed
from .context import ContextError, ContextManager
from .inference import Future




class Stream:
    """Handle of one generation run; resolved with the generated tokens."""

    _ids = itertools.count(1)

    def __init__(self, ctx_id: int, spec: SamplerSpec, max_tokens: int, stop: Sequence[int],
                 first_position: int):
        self.id = next(Stream._ids)
        self.ctx_id, self.spec, self.max_tokens = ctx_id, spec, max_tokens
        self.stop = frozenset(int(t) for t in stop)
        self.done = Future()
        self.tokens: List[int] = []          # generated tokens, first one comes from the prefill pass
        self.stamps: List[float] = []        # host time at which each token became visible
        self.first_position = first_position  # position of the first generated token when fed back
        self.finished = False
        self.error: Optional[BaseException] = None
        self.listeners: List[Callable[[List[int]], None]] = []
        self.row = -1
        self.fed = 0                          # generated tokens whose KV has been written
        self.cancelled = False

    def cancel(self) -> None:
        self.cancelled = True


class DecodeCohort:
    def __init__(self, ctxm: ContextManager, page_size: int, max_rows: int, on_finish: Optional[Callable] = None,
                 reserve_chunk: int = 4):
        self.ctxm, self.ps, self.max_rows = ctxm, page_size, max_rows
        self.on_finish = on_finish
        self.reserve_chunk = reserve_chunk
        m = max_rows
        self.n = 0
        self.streams: List[Optional[Stream]] = [None] * m
        self.pos = np.zeros(m, np.int32)          # position of the next input token
        self.kvlen = np.zeros(m, np.int32)        # tokens with KV before the next step
        self.npages = np.zeros(m, np.int32)
        self.maxp = 64
        self.table = np.zeros((m, self.maxp), np.int32)
        self.temp = np.zeros(m, np.float32)
        self.topk = np.zeros(m, np.int32)
        self.topp = np.ones(m, np.float32)
        self.minp = np.zeros(m, np.float32)
        self.seed = np.zeros(m, np.int64)
        self.remaining = np.zeros(m, np.int32)    # tokens still to generate (after those already sampled)
        self.prev_row = np.full(m, -1, np.int32)  # row in the layout of the step in flight, -1 = host token
        self.host_tok = np.zeros(m, np.int32)
        self.pending: List[tuple] = []            # (stream, first token) waiting to join
        self.lock = threading.Lock()
        self.rng = np.random.default_rng(7)
        self.steps = 0
        self.stop_union = np.zeros(0, np.int32)

    # ------------------------------------------------------------------ membership
    def has_work(self) -> bool:
        return self.n > 0 or bool(self.pending)

    def add(self, stream: Stream, first_token: int) -> None:
        """A stream's prefill finished with `first_token` sampled; it joins at the next step."""
        with self.lock:
            self.pending.append((stream, int(first_token)))

    def _grow_table(self, need: int) -> None:
        if need <= self.maxp:
            return
        new = max(need, self.maxp * 2)
        t = np.zeros((self.max_rows, new), np.int32)
        t[:, :self.maxp] = self.table
        self.table, self.maxp = t, new

    def _join(self, st: Stream, tok: int) -> bool:
        now = time.perf_counter()
        st.tokens.append(tok)
        st.stamps.append(now)
        for cb in st.listeners:
            cb([tok])
        if st.cancelled or st.max_tokens <= 1 or tok in st.stop:
            self._finish(st)
            return False
        try:
            pinned = self.ctxm.pin(st.ctx_id, 1)
        except ContextError as e:
            try:
                self.ctxm.reserve_working_pages(st.ctx_id, 1)
                pinned = self.ctxm.pin(st.ctx_id, 1)
            except ContextError:
                st.error = e
                self._finish(st)
                return False
        i = self.n
        self.n += 1
        self.streams[i] = st
        st.row = i
        self._grow_table(len(pinned.pages) + self.reserve_chunk)
        self.npages[i] = len(pinned.pages)
        self.table[i, :len(pinned.pages)] = pinned.pages
        self.kvlen[i] = pinned.kv_len
        self.pos[i] = st.first_position
        sp = st.spec
        self.temp[i] = sp.temperature
        self.topk[i] = sp.top_k if sp.kind in (SamplerKind.TOP_K, SamplerKind.TOP_K_TOP_P) else 0
        self.topp[i] = sp.top_p if sp.kind in (SamplerKind.TOP_P, SamplerKind.TOP_K_TOP_P) else 1.0
        self.minp[i] = sp.min_p if sp.kind == SamplerKind.MIN_P else 0.0
        self.seed[i] = sp.seed
        self.remaining[i] = st.max_tokens - 1
        self.prev_row[i] = -1
        self.host_tok[i] = tok
        if st.stop:
            self.stop_union = np.union1d(self.stop_union, np.fromiter(st.stop, np.int32)).astype(np.int32)
        return True

    def _remove_row(self, i: int) -> None:
        last = self.n - 1
        if i != last:
            for a in (self.pos, self.kvlen, self.npages, self.temp, self.topk, self.topp, self.minp, self.seed,
                      self.remaining, self.prev_row, self.host_tok):
                a[i] = a[last]
            self.table[i] = self.table[last]
            self.streams[i] = self.streams[last]
            self.streams[i].row = i
        self.streams[last] = None
        self.n = last

    # ------------------------------------------------------------------ one step
    def build(self) -> Optional[tuple]:
        """Compose the next step. Returns (CohortStep, snapshot of row -> stream) or None."""
        with self.lock:
            pend, self.pending = self.pending, []
        for st, tok in pend:
            if self.n >= self.max_rows:
                with self.lock:
                    self.pending.append((st, tok))   # no row free yet: joins at a later step
                continue
            self._join(st, tok)
        n = self.n
        if n == 0:
            return None
        ps = self.ps
        # KV capacity: the step writes slot kvlen (0-based) of each row
        need = (self.kvlen[:n] + 1 + ps - 1) // ps
        short = np.flatnonzero(need > self.npages[:n])
        for i in short.tolist():
            st = self.streams[i]
            k = int(need[i] - self.npages[i])
            got = None
            for chunk in (max(k, self.reserve_chunk), k):
                try:
                    before = self.ctxm.working_page_count(st.ctx_id)
                    self.ctxm.reserve_working_pages(st.ctx_id, chunk)
                    ctx = self.ctxm.contexts[st.ctx_id]
                    got = ctx.working_pages[before:]
                    break
                except ContextError as e:
                    err = e
            if got is None:
                st.error = err
                st._fail = True
                continue
            self._grow_table(int(self.npages[i]) + len(got))
            self.table[i, self.npages[i]:self.npages[i] + len(got)] = got
            self.npages[i] += len(got)
        failed = [i for i in short.tolist() if getattr(self.streams[i], "_fail", False)]
        for i in sorted(failed, reverse=True):
            st = self.streams[i]
            self._finish(st)
            self._remove_row(i)
        n = self.n
        if n == 0:
            return None
        kv_after = self.kvlen[:n] + 1
        used = (kv_after + ps - 1) // ps
        indptr = np.zeros(n + 1, np.int32)
        np.cumsum(used, out=indptr[1:])
        cols = np.arange(self.maxp, dtype=np.int32)[None, :]
        indices = self.table[:n][cols < used[:, None]]
        seeds = np.where(self.seed[:n] != 0, position_seed(self.seed[:n], self.pos[:n]),
                         self.rng.integers(1, 2**62, n, dtype=np.int64))
        step = CohortStep(r=n, host_tokens=self.host_tok[:n].copy(), src_row=self.prev_row[:n].copy(),
                          positions=self.pos[:n].copy(), kv_lens=kv_after.astype(np.int32), page_indptr=indptr,
                          page_indices=indices, temperature=self.temp[:n].copy(), top_k=self.topk[:n].copy(),
                          top_p=self.topp[:n].copy(), min_p=self.minp[:n].copy(), seeds=seeds)
        snapshot = list(self.streams[:n])
        # the step is now in flight: its rows become the source rows of the following step
        self.prev_row[:n] = np.arange(n, dtype=np.int32)
        self.kvlen[:n] += 1
        self.pos[:n] += 1
        for st in snapshot:
            st.fed += 1
        self.steps += 1
        return step, snapshot

    def absorb(self, snapshot: List[Stream], tokens: np.ndarray) -> None:
        """Tokens of a finished step: record them, detect stops, retire finished streams."""
        now = time.perf_counter()
        n = len(snapshot)
        stop_hit = np.isin(tokens[:n], self.stop_union) if self.stop_union.size else np.zeros(n, bool)
        toks = tokens[:n].tolist()
        for i, st in enumerate(snapshot):
            if st.finished:
                continue          # retired while this (one step late) result was in flight
            t = toks[i]
            st.tokens.append(t)
            st.stamps.append(now)
            if st.listeners:
                for cb in st.listeners:
                    cb([t])
            row = st.row
            self.remaining[row] -= 1
            if self.remaining[row] <= 0 or st.cancelled or (stop_hit[i] and t in st.stop):
                self._finish(st)
                self._remove_row(row)

    # ------------------------------------------------------------------ retirement
    def _finish(self, st: Stream) -> None:
        if st.finished:
            return
        st.finished = True
        if st.row >= 0 or st.fed:
            # tokens with KV: the first `fed` generated tokens were fed back as inputs, except that
            # a step launched after the final token was sampled wrote one slot too many (discarded)
            kept = min(st.fed, len(st.tokens) - 1) if st.error is None else min(st.fed, len(st.tokens))
            toks = st.tokens[:kept]
            pos = list(range(st.first_position, st.first_position + kept))
            try:
                self.ctxm.append_working_tokens(st.ctx_id, toks, pos)
            except ContextError:
                pass
            if st.row >= 0:
                self.ctxm.unpin(st.ctx_id)
            st.kept = kept
        else:
            st.kept = 0
        if self.on_finish:
            self.on_finish(st)
        if st.error is not None:
            st.done.set(exc=st.error)
        else:
            st.done.set(st)

    def abort_all(self, exc: BaseException) -> None:
        with self.lock:
            pend, self.pending = self.pending, []
        for st, _ in pend:
            st.error = exc
            self._finish(st)
        for i in range(self.n - 1, -1, -1):
            st = self.streams[i]
            st.error = exc
            self._finish(st)
            self._remove_row(i)
