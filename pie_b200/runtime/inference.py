"""Inference service: the path from an inferlet's `forward-pass.execute` to a batch slot,
with pass-level speculative execution.

`submit()` pins the context (consistent page list + kv length), queues a `PendingRequest` on
the driver's batch scheduler and returns a future. When a pass finishes, the scheduler thread
appends the pass's input tokens to the context lineage, unpins, and - if the pass is a plain
one-token-sampler decode - immediately builds and submits the NEXT single-token pass from the
sampled token ("staged" pass) before the inferlet has even seen the result. The inferlet's
next real `execute()` then claims that already-running pass instead of paying the pin +
queue + batch-wait latency. A claim must match (context, token, position, sampler, no masks);
anything else abandons the staged pass.

Behavioural counterpart of runtime/src/inference.rs:187-234 (submit / try_hit) and
runtime/src/inference/speculator.rs:208-249 (try_hit), :370-546 (chain start / extension),
:573-612 (eligibility).
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from ..driver.schema import MEDIA_TOKEN_BASE, SamplerSpec, SlotOutput
from .context import ContextError, ContextManager, Deferred
from .scheduler import BatchScheduler, PendingRequest


_FUTURE_LOCK = threading.Lock()       # guards the rare slow paths of every Future (a waiter's event, late callbacks)


class Future:
    """Minimal thread-safe future with completion callbacks (usable from asyncio or threads). The
    event a blocking waiter needs is created only when somebody waits: most futures here are consumed
    through callbacks, hundreds per fire, and an Event with its condition and lock costs more than the
    rest of the object."""

    __slots__ = ("_ev", "_result", "_exc", "_cbs", "done_flag", "_defer_tries")

    def __init__(self):
        self._ev = None
        self._result = None
        self._exc = None
        self._cbs: Optional[List[Callable]] = None
        self.done_flag = False

    def set(self, result=None, exc: Optional[BaseException] = None) -> None:
        with _FUTURE_LOCK:
            if self.done_flag:
                return
            self._result, self._exc, self.done_flag = result, exc, True
            cbs, self._cbs = self._cbs, None
            ev = self._ev
        if ev is not None:
            ev.set()
        if cbs:
            for cb in cbs:
                cb(self)

    def add_done_callback(self, cb: Callable) -> None:
        with _FUTURE_LOCK:
            if not self.done_flag:
                if self._cbs is None:
                    self._cbs = [cb]
                else:
                    self._cbs.append(cb)
                return
        cb(self)

    def done(self) -> bool:
        return self.done_flag

    def result(self, timeout: Optional[float] = None):
        if not self.done_flag:
            with _FUTURE_LOCK:
                if not self.done_flag and self._ev is None:
                    self._ev = threading.Event()
                ev = self._ev
            if not self.done_flag and not ev.wait(timeout):
                raise TimeoutError("forward pass did not complete in time")
        if self._exc is not None:
            raise self._exc
        return self._result


@dataclass
class ForwardOutput:
    slots: List[SlotOutput]
    spec_tokens: List[int] = field(default_factory=list)
    spec_positions: List[int] = field(default_factory=list)
    staged_hit: bool = False
    accepted_drafts: int = 0


@dataclass
class _Staged:
    token: int
    position: int
    sampler: SamplerSpec
    future: Future
    claimed: bool = False
    abandoned: bool = False


def _same_sampler(a: SamplerSpec, b: SamplerSpec) -> bool:
    return (a.kind == b.kind and a.temperature == b.temperature and a.top_k == b.top_k
            and a.top_p == b.top_p and a.min_p == b.min_p and a.seed == b.seed)


class InferenceService:
    def __init__(self, ctxm: ContextManager, schedulers: Sequence[BatchScheduler], speculation_depth: int = 1):
        self.ctxm, self.schedulers = ctxm, list(schedulers)
        self.depth = speculation_depth
        self.cohorts: list = []       # DecodeCohort per driver (set by the engine)
        self.staged: Dict[int, _Staged] = {}
        self.lock = threading.Lock()
        self._recurrent: Optional[bool] = None      # the model has recurrent layers (set on first use)
        self.system_spec_tokens = 0  # > 0: the runtime drafts up to this many tokens per generator step (n-gram look-up)
        self.system_spec_ngram = 2
        self.max_defers = 64         # times one request may wait (restore queue, slot shortage) before it fails
        self.stats = {"system_spec_proposed": 0, "system_spec_accepted": 0, "submits": 0, "bypass_hits": 0, "chain_submits": 0, "chain_drops": 0,
                      "tokens_appended": 0}
        self.on_tokens: Optional[Callable[[int, int], None]] = None   # (context id, n tokens) accounting hook

    # ------------------------------------------------------------------ public
    def submit(self, cid: int, tokens: Sequence[int], positions: Sequence[int],
               samplers: Sequence[tuple], masks: Optional[list] = None, logit_mask: Optional[list] = None,
               spec_tokens: Sequence[int] = (), spec_positions: Sequence[int] = (), adapter: int = -1,
               speculate: bool = True, spec_budget: Optional[int] = None) -> Future:
        """Queue one forward pass of context `cid`; resolves to a ForwardOutput.

        `spec_budget`: the caller can take up to this many extra tokens from this pass (a generator step; None:
        it cannot). With system speculation on, the runtime then drafts continuation tokens itself, verifies
        them in the same pass and returns the accepted ones in `ForwardOutput.spec_tokens`."""
        self.stats["submits"] += 1
        tokens, positions = list(tokens), list(positions)
        if (self.system_spec_tokens > 0 and spec_budget and len(tokens) == 1 and len(samplers) == 1 and not spec_tokens
                and masks is None and logit_mask is None and adapter < 0 and samplers[0][0] == 0
                and samplers[0][1].is_token and speculate):
            drafted = self._system_draft(cid, tokens[0], positions[0], min(self.system_spec_tokens, spec_budget))
            if drafted:
                d_tokens, d_positions = drafted
                fut = Future()
                sp = samplers[0][1]
                inner = Future()

                def finish(f: Future, n=len(d_tokens)):
                    try:
                        out = f.result()
                    except BaseException as e:  # noqa: BLE001
                        fut.set(exc=e)
                        return
                    k = out.accepted_drafts
                    # slot i holds the successor of input row i: rows 1..k are the successors of accepted drafts
                    out.spec_tokens = [s.token for s in out.slots[1:k + 1]]
                    out.spec_positions = d_positions[:k]
                    out.system_drafts = n
                    out.slots = out.slots[:1]
                    self.stats["system_spec_proposed"] += n
                    self.stats["system_spec_accepted"] += k
                    fut.set(out)
                inner.add_done_callback(finish)
                prev = self._abandon(cid)
                args = (cid, tokens, positions, [(i, sp) for i in range(len(d_tokens) + 1)], None, None, d_tokens,
                        d_positions, -1, False, inner)
                if prev is not None and not prev.future.done():
                    prev.future.add_done_callback(lambda _f: self._start(*args))
                else:
                    self._start(*args)
                return fut
        hit = self._try_hit(cid, tokens, positions, samplers, masks, logit_mask, spec_tokens)
        if hit is not None:
            return hit
        prev = self._abandon(cid)
        fut = Future()
        args = (cid, tokens, positions, list(samplers), masks, logit_mask, list(spec_tokens),
                list(spec_positions), adapter, speculate, fut)
        if prev is not None and not prev.future.done():
            # the abandoned pass still writes the tail slot: run the real pass after it
            prev.future.add_done_callback(lambda _f: self._start(*args))
        else:
            self._start(*args)
        return fut

    def drop_context(self, cid: int) -> None:
        self._abandon(cid)

    def _system_draft(self, cid: int, token: int, position: int, k: int):
        """Prompt-look-up drafter: find the most recent earlier occurrence of the context's last `n` tokens
        (ending with the token about to be fed) and propose what followed it. Returns (tokens, positions) or
        None; also makes sure the context has page capacity for the drafts (else no draft)."""
        ctx = self.ctxm.contexts.get(cid)
        if ctx is None or k <= 0 or self.ctxm.rs[ctx.driver].supported:
            return None
        hist = list(ctx.committed_tokens) + list(ctx.tokens) + [token]
        n = self.system_spec_ngram
        if len(hist) <= n:
            return None
        key = hist[-n:]
        found = -1
        for i in range(len(hist) - n - 1, -1, -1):           # newest match first
            if hist[i:i + n] == key:
                found = i + n
                break
        if found < 0 or found >= len(hist):
            return None
        drafts = hist[found:found + k]
        for j, t in enumerate(drafts):          # a media placeholder is never a sampled token: the draft ends before it
            if t >= MEDIA_TOKEN_BASE:
                drafts = drafts[:j]
                break
        if not drafts:
            return None
        ps = self.ctxm.page_size
        need = self.ctxm.kv_len(cid) + 1 + len(drafts) + 1
        have = (len(ctx.chain) + len(ctx.working_pages)) * ps
        if need > have:
            try:
                self.ctxm.reserve_working_pages(cid, -(-(need - have) // ps))
            except ContextError:
                return None
        return drafts, [position + 1 + i for i in range(len(drafts))]

    def start_stream(self, cid: int, tokens: Sequence[int], positions: Sequence[int], spec: SamplerSpec,
                     max_tokens: int, stop: Sequence[int] = ()):
        """Plain generation offloaded to the runtime: one ordinary pass over `tokens` that samples
        the first token, then the context decodes inside the driver's cohort (array-form,
        device-fed tokens) until `max_tokens` or a stop token. Returns a cohort Stream."""
        from .cohort import Stream
        stream = Stream(cid, spec, max_tokens, stop, first_position=int(positions[-1]) + 1)
        driver = self.ctxm.contexts[cid].driver
        fut = self.submit(cid, tokens, positions, [(len(tokens) - 1, spec)], speculate=False)

        def first(f: Future):
            try:
                out = f.result()
            except BaseException as e:  # noqa: BLE001
                stream.error = e
                stream.finished = True
                stream.done.set(exc=e)
                return
            self.cohorts[driver].add(stream, out.slots[0].token)

        fut.add_done_callback(first)
        return stream

    # ------------------------------------------------------------------ staged passes
    def _try_hit(self, cid, tokens, positions, samplers, masks, logit_mask, spec_tokens) -> Optional[Future]:
        with self.lock:
            st = self.staged.get(cid)
            if st is None or st.claimed or st.abandoned:
                return None
            ok = (len(tokens) == 1 and tokens[0] == st.token and positions[0] == st.position
                  and masks is None and logit_mask is None and not spec_tokens and len(samplers) == 1
                  and samplers[0][0] == 0 and _same_sampler(samplers[0][1], st.sampler))
            if not ok:
                return None
            st.claimed = True
            parked = getattr(st, "_parked", None) is not None
            self.stats["bypass_hits"] += 1
        out = Future()

        def relay(f: Future):
            try:
                res = f.result()
            except BaseException as e:  # noqa: BLE001
                out.set(exc=e)
                return
            res.staged_hit = True
            out.set(res)

        # if the pass already finished, finalise it now (lineage append + next stage)
        if parked:
            self._finalise_staged(cid, st)
        st.future.add_done_callback(relay)
        return out

    def _abandon(self, cid: int) -> Optional[_Staged]:
        with self.lock:
            st = self.staged.get(cid)
            if st is None:
                return None
            if st.claimed and not st.future.done():
                return st   # claimed pass in flight: the caller must order after it
            del self.staged[cid]
            parked = False
            if not st.claimed:
                st.abandoned = True
                parked = getattr(st, "_parked", None) is not None
                st._parked = None
                self.stats["chain_drops"] += 1
        if parked:
            self.ctxm.unpin(cid)
        return st

    # ------------------------------------------------------------------ execution
    def _start(self, cid, tokens, positions, samplers, masks, logit_mask, spec_tokens, spec_positions,
               adapter, speculate, fut: Future, staged: Optional[_Staged] = None) -> None:
        all_tokens = tokens + spec_tokens
        all_positions = positions + spec_positions
        try:
            pinned = self.ctxm.pin(cid, len(all_tokens))
        except Deferred as e:
            # evicted and no room to come back yet: wait in the restore queue, bounded by the deadline
            tries = getattr(fut, "_defer_tries", 0)
            if tries >= self.max_defers:
                fut.set(exc=e)
                return
            fut._defer_tries = tries + 1
            self.stats["deferred_starts"] = self.stats.get("deferred_starts", 0) + 1
            retry = lambda: self._start(cid, tokens, positions, samplers, masks, logit_mask, spec_tokens,
                                        spec_positions, adapter, speculate, fut, staged)
            try:
                ctx = self.ctxm.contexts.get(cid)
                if ctx is not None and ctx.state.value != "suspended":
                    # resident but short of something another context holds (a recurrent-state slot, pages):
                    # try again when a context is unpinned or gives pages back
                    self.ctxm.on_pages_freed(ctx.driver, retry)
                else:
                    self.ctxm.when_restorable(cid, retry)
            except ContextError as e2:
                fut.set(exc=e2)
            return
        except ContextError as e:
            fut.set(exc=e)
            return
        # a context restored from eviction must first replay the KV it lost
        replay = self.ctxm.take_pending_replay(cid)
        sched = self.schedulers[pinned.driver]
        if replay:
            self._replay_then(cid, pinned, replay, lambda: self._queue(
                sched, cid, pinned, all_tokens, all_positions, samplers, masks, logit_mask, len(spec_tokens),
                adapter, speculate, fut, staged, len(tokens)))
            return
        self._queue(sched, cid, pinned, all_tokens, all_positions, samplers, masks, logit_mask,
                    len(spec_tokens), adapter, speculate, fut, staged, len(tokens))

    def _replay_then(self, cid, pinned, spans, then: Callable) -> None:
        """Rebuild lost KV by re-running the lineage as forward passes without samplers."""
        sched = self.schedulers[pinned.driver]
        spans = list(spans)

        reset = [pinned.rs_reset]        # the first replayed span starts the recurrent state over

        def step(_res=None):
            if isinstance(_res, Exception) or not spans:
                then()
                return
            toks, poss, first = spans.pop(0)
            sched.submit(PendingRequest(context_id=cid, tokens=toks, positions=poss, pages=pinned.pages,
                                        kv_len=first, samplers=[], on_done=step, rs_slot=pinned.rs_slot,
                                        rs_reset=reset[0]))
            reset[0] = 0
        pinned.rs_reset = 0                # ... and the pass that follows the replay continues from it
        step()

    def _queue(self, sched, cid, pinned, tokens, positions, samplers, masks, logit_mask, n_spec, adapter,
               speculate, fut, staged, n_plain) -> None:
        def on_done(result):
            self._on_done(cid, tokens, positions, samplers, masks, logit_mask, n_spec, n_plain, speculate,
                          fut, staged, result)

        sched.submit(PendingRequest(context_id=cid, tokens=tokens, positions=positions, pages=pinned.pages,
                                    kv_len=pinned.kv_len, samplers=list(samplers), masks=masks,
                                    logit_mask=logit_mask, spec_count=n_spec, adapter=adapter, on_done=on_done,
                                    rs_slot=pinned.rs_slot, rs_reset=pinned.rs_reset))

    def _on_done(self, cid, tokens, positions, samplers, masks, logit_mask, n_spec, n_plain, speculate, fut,
                 staged, result) -> None:
        """Runs on the scheduler thread right after the batch returned."""
        if isinstance(result, Exception):
            self.ctxm.unpin(cid)
            fut.set(exc=result)
            return
        out = ForwardOutput(slots=list(result))
        out.driver_accepted = getattr(result, "spec_accepted", None)
        if staged is not None:
            # Lock order: the context manager's lock may be held when this lock is taken (the scheduler
            # scatters a whole fire under it), never the other way round - so no call into the context
            # manager from inside `with self.lock`.
            park = abandoned = False
            with self.lock:
                if staged.abandoned:
                    abandoned = True
                elif not staged.claimed:
                    # finished before anybody asked for it: park the result, keep the pin
                    staged._parked = (tokens, positions, samplers, out)
                    park = True
            if abandoned:
                self.ctxm.unpin(cid)
                fut.set(out)
                return
            if park:
                fut.set(out)
                return
        accepted = self._accept(tokens, positions, samplers, n_spec, n_plain, out)
        self._append_and_unpin(cid, tokens[:accepted], positions[:accepted], masks)
        if staged is not None:
            with self.lock:
                if self.staged.get(cid) is staged:
                    del self.staged[cid]
        if speculate and self.depth > 0:
            self._maybe_stage(cid, tokens, positions, samplers, masks, logit_mask, n_spec, out)
        fut.set(out)

    def _finalise_staged(self, cid: int, st: _Staged) -> None:
        """A parked (finished, unclaimed) pass was just claimed."""
        parked = getattr(st, "_parked", None)
        if parked is None:
            return
        tokens, positions, samplers, out = parked
        st._parked = None
        with self.ctxm.lock:          # one hold for the append, the unpin and the next stage's pin
            self._append_and_unpin(cid, tokens, positions, None)
            with self.lock:
                if self.staged.get(cid) is st:
                    del self.staged[cid]
            if self.depth > 0:
                self._maybe_stage(cid, tokens, positions, samplers, None, None, 0, out)

    def _accept(self, tokens, positions, samplers, n_spec, n_plain, out: ForwardOutput) -> int:
        """Number of input tokens whose KV is kept. Draft tokens are kept while the token sampled
        at the previous row equals the draft; the response tokens become accepted drafts + bonus."""
        if n_spec == 0:
            return len(tokens)
        verdict = getattr(out, "driver_accepted", None)
        if verdict is not None:                 # the driver compared drafts and samples itself
            out.accepted_drafts = min(int(verdict), n_spec)
            self.stats["driver_verified"] = self.stats.get("driver_verified", 0) + 1
            return n_plain + out.accepted_drafts
        # samplers attached at rows n_plain-1 .. n_plain-1+n_spec verify the drafts in order
        by_row = {idx: k for k, (idx, sp) in enumerate(samplers) if sp.is_token}
        accepted = 0
        row = n_plain - 1
        for j in range(n_spec):
            k = by_row.get(row + j)
            if k is None or out.slots[k].token != tokens[n_plain + j]:
                break
            accepted += 1
        out.accepted_drafts = accepted
        return n_plain + accepted

    def _append_and_unpin(self, cid, tokens, positions, masks) -> None:
        try:
            keys = None
            if masks is not None:
                keys = [b"m" + bytes(str(m), "ascii") for m in masks[:len(tokens)]]
            self.ctxm.append_working_tokens(cid, tokens, positions, keys)
            self.stats["tokens_appended"] += len(tokens)
            if self.on_tokens:
                self.on_tokens(cid, len(tokens))
        except ContextError:
            pass
        self.ctxm.unpin(cid)

    def _maybe_stage(self, cid, tokens, positions, samplers, masks, logit_mask, n_spec, out) -> None:
        """Eligibility: exactly one token-sampler slot at the last input row, no masks, no drafts."""
        if masks is not None or logit_mask is not None or n_spec or len(samplers) != 1:
            return
        if self._recurrent is None:
            self._recurrent = any(rs.supported for rs in self.ctxm.rs)
        if self._recurrent:
            return  # a staged pass that is later abandoned would already have advanced the recurrent state
        idx, sp = samplers[0]
        if idx != len(tokens) - 1 or not sp.is_token or out.slots[0].kind != "token":
            return
        nxt_tok, nxt_pos = out.slots[0].token, positions[-1] + 1
        try:
            pinned = self.ctxm.pin(cid, 1)
        except ContextError:
            return  # no free slot at the tail (or context gone): the inferlet will reserve and submit
        fut = Future()
        st = _Staged(nxt_tok, nxt_pos, sp, fut)
        with self.lock:
            taken = cid in self.staged
            if not taken:
                self.staged[cid] = st
        if taken:
            self.ctxm.unpin(cid)
            return
        self.stats["chain_submits"] += 1
        sched = self.schedulers[pinned.driver]
        self._queue(sched, cid, pinned, [nxt_tok], [nxt_pos], [(0, sp)], None, None, 0, -1, True, fut, st, 1)
