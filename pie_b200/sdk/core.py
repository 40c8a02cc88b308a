"""Inferlet SDK core: Model, Tokenizer, Context, Forward, Output, Generator, GenStep.

Three layers, as in the reference SDKs (sdk/python/src/inferlet/{context,forward,generation}.py;
sdk/rust/inferlet/src/{context.rs:82-778, forward.rs:104-531, generation.rs:58-860}):

* Context   - KV cache handle + pending-token buffer + chat fillers + fork/save/open/take.
* Forward   - one forward pass with automatic page reserve/commit, samplers, probes, masks,
              speculative drafts.
* Generator - multi-step decode state machine over Forward (max tokens, stop tokens,
              constraints, custom speculators).

Decode-loop shape: the token sampled at step k is the single input of step k+1 at position
seq_len, sampled at index 0 (generation.rs:315-375). flush() = forward without a sampler,
then commit of floor(tokens / page) pages (context.rs:407-455).
"""
from __future__ import annotations

import asyncio
import json
from typing import Any, Iterable, List, Optional, Sequence

from ..driver.schema import SamplerSpec
from ..runtime import brle
from ..runtime.context import Deferred as _Deferred
from . import host
from .sample import Distribution, Entropy, Logits, Logprob, Logprobs, Sampler


class Tokenizer:
    def __init__(self, impl):
        self._t = impl

    def encode(self, text: str) -> List[int]:
        return list(self._t.encode(text))

    def decode(self, tokens: Sequence[int]) -> str:
        return self._t.decode(list(tokens))

    def vocabs(self):
        return self._t.vocabs()

    def split_regex(self) -> str:
        return getattr(self._t, "split_regex", lambda: "")()

    def special_tokens(self):
        return getattr(self._t, "special_tokens", lambda: ([], []))()

    @property
    def eos_tokens(self) -> List[int]:
        return list(getattr(self._t, "eos_tokens", []))


class Model:
    def __init__(self, name: str):
        self.name = name
        self._entry = host.engine().model(name)

    @staticmethod
    def load(name: Optional[str] = None) -> "Model":
        eng = host.engine()
        return Model(name if name is not None else next(iter(eng.models)))

    def tokenizer(self) -> Tokenizer:
        if self._entry.tokenizer is None:
            raise RuntimeError(f"model {self.name} has no tokenizer")
        return Tokenizer(self._entry.tokenizer)

    @property
    def instruct(self):
        return self._entry.instruct

    def default_system_speculation(self) -> bool:
        return bool(self._entry.caps[0].system_speculation)

    @property
    def page_size(self) -> int:
        return self._entry.page_size

    def __repr__(self) -> str:
        return f"Model({self.name!r})"


class SampleHandle:
    def __init__(self, slot: int, count: int):
        self.slot, self.count = slot, count


class ProbeHandle:
    def __init__(self, slot: int, kind: str):
        self.slot, self.kind = slot, kind


class Output:
    """Typed access to the per-slot results of one forward pass."""

    def __init__(self, raw, slot_map):
        self._raw, self._map = raw, slot_map
        self.tokens: List[int] = []          # tokens accepted by this step (Generator fills it)

    @property
    def raw(self):
        return self._raw

    def token(self, h: SampleHandle) -> Optional[int]:
        s = self._raw.slots[h.slot]
        return s.token if s.kind == "token" else None

    def tokens_at(self, h: SampleHandle) -> List[int]:
        return [self._raw.slots[h.slot + i].token for i in range(h.count)]

    def distribution(self, h: ProbeHandle):
        s = self._raw.slots[h.slot]
        return (s.ids, s.probs) if s.kind == "distribution" else None

    def logits(self, h: ProbeHandle) -> Optional[bytes]:
        s = self._raw.slots[h.slot]
        return s.logits if s.kind == "logits" else None

    def logprobs(self, h: ProbeHandle) -> Optional[List[float]]:
        s = self._raw.slots[h.slot]
        return s.logprobs if s.kind == "logprobs" else None

    def entropy(self, h: ProbeHandle) -> Optional[float]:
        s = self._raw.slots[h.slot]
        return s.entropy if s.kind == "entropy" else None

    @property
    def accepted_drafts(self) -> int:
        return getattr(self._raw, "accepted_drafts", 0)


class Forward:
    """One forward pass over a context, with automatic working-page management."""

    def __init__(self, ctx: "Context"):
        self.ctx = ctx
        self._tokens: List[int] = []
        self._positions: List[int] = []
        self._samplers: List[tuple] = []      # (index, SamplerSpec)
        self._mask: Optional[List[int]] = None
        self._attn_masks: Optional[List[List[int]]] = None
        self._spec_tokens: List[int] = []
        self._spec_positions: List[int] = []
        self._adapter = -1
        self._speculate = True

    @property
    def start_position(self) -> int:
        return self.ctx.seq_len

    def input(self, tokens: Sequence[int]) -> "Forward":
        start = self.ctx.seq_len + len(self._tokens)
        self._tokens.extend(int(t) for t in tokens)
        self._positions.extend(range(start, start + len(tokens)))
        return self

    def input_at(self, tokens: Sequence[int], positions: Sequence[int]) -> "Forward":
        self._tokens.extend(int(t) for t in tokens)
        self._positions.extend(int(p) for p in positions)
        return self

    def speculative(self, tokens: Sequence[int], positions: Optional[Sequence[int]] = None) -> "Forward":
        """Attach draft tokens to be verified in this pass (WIT input-speculative-tokens)."""
        start = (self._positions[-1] + 1) if self._positions else self.ctx.seq_len
        self._spec_tokens = [int(t) for t in tokens]
        self._spec_positions = list(positions) if positions is not None else list(range(start, start + len(tokens)))
        return self

    def sample(self, indices: Sequence[int], sampler: Sampler) -> SampleHandle:
        h = SampleHandle(len(self._samplers), len(indices))
        for i in indices:
            self._samplers.append((int(i), sampler.spec))
        return h

    def probe(self, index: int, probe: Any) -> ProbeHandle:
        spec: SamplerSpec = probe.spec
        h = ProbeHandle(len(self._samplers), spec.kind.name.lower())
        self._samplers.append((int(index), spec))
        return h

    def mask(self, mask: Sequence[int]) -> "Forward":
        """Vocabulary mask (BRLE) applied to every sampler of this pass; masks AND together."""
        self._mask = list(mask) if self._mask is None else brle.logical_and(self._mask, mask)
        return self

    def attention_mask(self, masks: Sequence[Sequence[int]]) -> "Forward":
        self._attn_masks = [list(m) for m in masks]
        return self

    def adapter(self, adapter) -> "Forward":
        self._adapter = getattr(adapter, "id", -1)
        return self

    def pass_speculation(self, flag: bool) -> "Forward":
        self._speculate = flag
        return self

    async def execute(self) -> Output:
        ctx = self.ctx
        n_in = len(self._tokens) + len(self._spec_tokens)
        if n_in == 0:
            from ..runtime.inference import ForwardOutput
            return Output(ForwardOutput(slots=[]), None)
        try:
            ctx._reserve_for(n_in)                       # the common case needs no waiting (and no coroutine)
        except _Deferred:
            await ctx._reserve_async(n_in)
        if ctx.__dict__.get("_pending_media"):
            await ctx._await_media()
        svc = ctx._entry.inference
        fut = svc.submit(ctx.id, self._tokens, self._positions, self._samplers, self._attn_masks, self._mask,
                         self._spec_tokens, self._spec_positions, self._adapter, self._speculate,
                         spec_budget=getattr(self, "_spec_budget", None))
        raw = await host.wait(fut)
        accepted = len(self._tokens) + getattr(raw, "accepted_drafts", 0)
        drafted = self._spec_positions if self._spec_positions else list(getattr(raw, "spec_positions", ()))
        ctx._after_pass(accepted, self._positions + drafted)
        return Output(raw, None)


class Context:
    """Handle on one KV context of the calling process (WIT resource `context`)."""

    def __init__(self, model: Model, _id: Optional[int] = None, _seq_len: int = 0, _next_pos: int = 0):
        self._model = model
        self._entry = model._entry
        self._p = host.proc()
        self.id = self._entry.ctxm.create(self._p.id) if _id is None else _id
        self._buffer: List[int] = []
        self._seq_len = _seq_len          # tokens whose KV exists
        self._next_pos = _next_pos
        self._released = False

    # ---- constructors
    @classmethod
    def open(cls, model: Model, name: str) -> Optional["Context"]:
        p = host.proc()
        try:
            cid = model._entry.ctxm.open(p.username, name, p.id)
        except Exception:
            return None
        return cls._adopt(model, cid)

    @classmethod
    def take(cls, model: Model, name: str) -> Optional["Context"]:
        p = host.proc()
        try:
            cid = model._entry.ctxm.take(p.username, name, p.id)
        except Exception:
            return None
        return cls._adopt(model, cid)

    @classmethod
    def _adopt(cls, model: Model, cid: int) -> "Context":
        n = model._entry.ctxm.kv_len(cid)
        c = model._entry.ctxm.contexts[cid]
        last = max([c.max_committed_position] + c.positions) if (c.positions or c.chain) else -1
        return cls(model, _id=cid, _seq_len=n, _next_pos=last + 1)

    @staticmethod
    def delete(model: Model, name: str) -> None:
        model._entry.ctxm.delete_snapshot(host.proc().username, name)

    def fork(self) -> "Context":
        cid = self._entry.ctxm.fork(self.id)
        c = Context(self._model, _id=cid, _seq_len=self._seq_len, _next_pos=self._next_pos)
        c._buffer = list(self._buffer)
        if self.__dict__.get("_pending_media"):
            c._pending_media = list(self._pending_media)
        if self.__dict__.get("_bidir_spans"):
            c._bidir_spans = list(self._bidir_spans)
        return c

    def save(self, name: str) -> None:
        self._entry.ctxm.save(self.id, self._p.username, name)

    def snapshot(self) -> str:
        return self._entry.ctxm.snapshot(self.id, self._p.username)

    def release(self) -> None:
        if not self._released:
            self._released = True
            self._entry.inference.drop_context(self.id)
            self._entry.ctxm.destroy(self.id)

    destroy = release

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.release()

    # ---- properties
    @property
    def model(self) -> Model:
        return self._model

    @property
    def page_size(self) -> int:
        return self._entry.page_size

    @property
    def seq_len(self) -> int:
        return self._next_pos

    @property
    def kv_len(self) -> int:
        return self._seq_len

    @property
    def buffer(self) -> List[int]:
        return list(self._buffer)

    def committed_page_count(self) -> int:
        return self._entry.ctxm.committed_page_count(self.id)

    def working_page_count(self) -> int:
        return self._entry.ctxm.working_page_count(self.id)

    # ---- fillers
    def _fill(self, role: str, message: str) -> "Context":
        ins = self._model.instruct
        tok = self._model.tokenizer()
        if ins is None:
            self._buffer.extend(tok.encode(message))
            return self
        if ins.fold_system:
            # no system role in this family: hold the text and open the next user turn with it
            if role == "system":
                self._held_system = (getattr(self, "_held_system", "") + message + "\n")
                return self
            if role == "user" and getattr(self, "_held_system", ""):
                message, self._held_system = self._held_system + message, ""
        self._buffer.extend(ins.render(role, message, tok, first=self.seq_len + len(self._buffer) == 0))
        return self

    def system(self, message: str) -> "Context":
        return self._fill("system", message)

    def user(self, message: str) -> "Context":
        return self._fill("user", message)

    def assistant(self, message: str) -> "Context":
        return self._fill("assistant", message)

    def cue(self) -> "Context":
        ins = self._model.instruct
        if ins is not None:
            if getattr(self, "_held_system", ""):          # a system text with no user turn after it
                held, self._held_system = self._held_system, ""
                self._fill("user", held.rstrip("\n"))
            self._buffer.extend(ins.cue(self._model.tokenizer()))
        return self

    def seal(self) -> "Context":
        ins = self._model.instruct
        if ins is not None:
            self._buffer.extend(ins.seal(self._model.tokenizer()))
        return self

    def append(self, tokens: Iterable[int]) -> "Context":
        self._buffer.extend(int(t) for t in tokens)
        return self

    def _append_clip(self, kind: str, features) -> "Context":
        from . import media
        media.require(self._model, kind)
        reg = self._entry.media
        # the driver encodes the clip (once per distinct content, on the registry's worker thread) and keeps the result
        # on the device; the context takes one placeholder token per encoder row at once, which the request builder
        # turns into media spans, and its next forward pass waits for the encoder
        toks, entry = reg.put(self.id, kind, features.patches, [features.grid], features.num_tokens)
        spec = getattr(self._entry.caps[0], "media_spec", None) or {}
        before, after = (spec.get("delimiters") or {}).get(kind, ("", ""))
        if self._entry.tokenizer is None:       # token-level use without a tokenizer: the caller places any markers itself
            before = after = ""
        if before:          # the model's own span markers go around the clip
            self._buffer.extend(self._model.tokenizer().encode(before))
        if spec.get("bidirectional") and kind in ("image", "video"):
            # the rows of one image see each other in both directions: remembered as spans of the pending buffer, and
            # run with attention masks before anything else consumes the buffer (`_flush_media_spans`)
            frames = max(1, int(features.grid[0]))
            per = len(toks) // frames
            spans = self.__dict__.setdefault("_bidir_spans", [])
            spans.extend((len(self._buffer) + f * per, per) for f in range(frames))
        self._buffer.extend(toks)
        if after:
            self._buffer.extend(self._model.tokenizer().encode(after))
        if not entry.ready.done():
            self.__dict__.setdefault("_pending_media", []).append(entry)
        else:
            entry.ready.result()            # an encoder error of an earlier caller is this caller's too
        return self

    async def _flush_media_spans(self) -> None:
        """Run the pending buffer up to the end of its last bidirectional span through the model: the text before and
        between spans in ordinary causal passes, every span in a pass of its own whose rows see every key up to the span's
        end (attention masks; the scheduler keeps such a pass in one fire). What follows the last span stays pending."""
        spans = sorted(self.__dict__.get("_bidir_spans") or ())
        if not spans:
            return
        self._bidir_spans = []
        buf, pos = self._buffer, 0
        self._buffer = buf[spans[-1][0] + spans[-1][1]:]
        for s, n in spans:
            if s > pos:
                await Forward(self).input(buf[pos:s]).execute()
            hi = self._seq_len + n
            await Forward(self).input(buf[s:s + n]).attention_mask([[0, hi]] * n).execute()
            pos = s + n

    async def _await_media(self) -> None:
        """Clips appended since the last pass: every path that submits this context's tokens waits here until their
        encoders are done (and gets an encoder's error)."""
        pending = self.__dict__.get("_pending_media")
        while pending:
            await host.wait(pending.pop().ready)

    def append_image(self, image) -> "Context":
        """Splice an image into the context: one placeholder token per row of the vision encoder's output
        (needs a driver with a vision encoder). Chat markers around the image are the template's business."""
        return self._append_clip("image", image.features)

    def append_audio(self, audio) -> "Context":
        """Splice an audio clip into the context: one placeholder token per 40 ms (needs a driver with an audio encoder)."""
        return self._append_clip("audio", audio)

    def append_video(self, video) -> "Context":
        return self._append_clip("video", video.features)

    # ---- page management
    def _reserve_for(self, n_new: int) -> None:
        ctxm, ps = self._entry.ctxm, self.page_size
        have = (ctxm.committed_page_count(self.id) + ctxm.working_page_count(self.id)) * ps
        # one token of slack keeps a tail slot free for the runtime's staged (speculative) pass
        need = self._seq_len + n_new + 1
        if need > have:
            ctxm.reserve_working_pages(self.id, -(-(need - have) // ps))

    async def _reserve_async(self, n_new: int, timeout_s: float = 120.0) -> None:
        """`_reserve_for` that waits while the allocation is deferred (pages held for, or only obtainable
        from, contexts that outrank this one): it retries whenever pages are given back, until the
        deadline, then fails with the deferral (runtime/src/context/sched.rs:717 `when_allocated`)."""
        import time as _time
        from ..runtime.context import Deferred
        from ..runtime.inference import Future
        deadline = _time.monotonic() + timeout_s
        while True:
            try:
                return self._reserve_for(n_new)
            except Deferred:
                if _time.monotonic() >= deadline:
                    raise
                ctxm = self._entry.ctxm
                fut = Future()
                ctxm.on_pages_freed(ctxm.contexts[self.id].driver, lambda: fut.done_flag or fut.set(True))
                try:
                    await asyncio.wait_for(host.wait(fut), timeout=min(1.0, max(0.01, deadline - _time.monotonic())))
                except asyncio.TimeoutError:
                    pass

    def _after_pass(self, accepted: int, positions: Sequence[int]) -> None:
        before = self._seq_len
        self._seq_len += accepted
        if accepted:
            self._next_pos = max(self._next_pos, positions[accepted - 1] + 1)
        ps = self.page_size
        if before // ps == self._seq_len // ps and not getattr(self, "_commit_retry", False):
            return  # committed pages are full ones: a working page fills only when a page boundary is crossed
        ctxm = self._entry.ctxm
        full = ctxm.working_page_token_count(self.id) // ps
        if full:
            try:
                ctxm.commit_working_pages(self.id, full)
                self._commit_retry = False
            except Exception:
                self._commit_retry = True  # non-monotonic positions (custom layouts) stay in working pages

    async def flush(self) -> None:
        """Run the pending tokens through the model without sampling."""
        if self.__dict__.get("_bidir_spans"):
            await self._flush_media_spans()
        if not self._buffer:
            return
        toks, self._buffer = self._buffer, []
        await Forward(self).input(toks).execute()

    def truncate(self, n: int) -> None:
        """Drop the last n tokens of the working tail."""
        n = min(n, self._entry.ctxm.working_page_token_count(self.id))
        self._entry.inference.drop_context(self.id)
        self._entry.ctxm.truncate_working_page_tokens(self.id, n)
        self._seq_len -= n
        self._next_pos -= n

    def forward(self) -> Forward:
        return Forward(self)

    def generate(self, sampler: Sampler, max_tokens: Optional[int] = None, stop: Optional[Iterable[int]] = None,
                 constrain=None, logit_mask: Optional[Sequence[int]] = None, **kw) -> "Generator":
        g = Generator(self, sampler, **kw)
        if max_tokens is not None:
            g.max_tokens(max_tokens)
        if stop is not None:
            g.stop(stop)
        if constrain is not None:
            for c in (constrain if isinstance(constrain, (list, tuple)) else [constrain]):
                g.constrain(c)
        if logit_mask is not None:
            from .grammar import StaticMaskConstraint
            g.constrain(StaticMaskConstraint(logit_mask))
        return g

    def set_bid(self, value: float) -> None:
        self._entry.ctxm.set_bid(self.id, value)

    def suspend(self) -> None:
        self._entry.inference.drop_context(self.id)
        self._entry.ctxm.suspend(self.id)


class GenStep:
    """One step of a Generator: a prepared Forward that the caller may extend with probes."""

    def __init__(self, gen: "Generator", fwd: Forward, handle: SampleHandle, n_draft: int):
        self.gen, self.forward, self.handle, self.n_draft = gen, fwd, handle, n_draft

    def probe(self, index: int, probe: Any) -> ProbeHandle:
        return self.forward.probe(index, probe)

    async def execute(self) -> Output:
        out = await self.forward.execute()
        sampled = out.tokens_at(self.handle)
        if self.n_draft:
            k = out.accepted_drafts
            accepted = sampled[: k + 1]        # accepted drafts' successors + bonus token
        else:
            # the runtime may have drafted and verified a continuation itself (system speculation)
            accepted = sampled[:1] + list(getattr(out.raw, "spec_tokens", ()) or [])
        out.tokens = self.gen.accept(accepted)
        extra = len(accepted) - len(out.tokens)
        if extra > 0 and not self.n_draft:
            try:                               # the generator stopped inside the accepted run: drop the KV beyond it
                self.gen.ctx.truncate(extra)
            except Exception:  # noqa: BLE001
                pass
        return out


class Generator:
    """Multi-step decode loop. `async for step in gen: out = await step.execute()`."""

    def __init__(self, ctx: Context, sampler: Sampler, speculator=None, adapter=None):
        self.ctx, self.sampler, self.speculator = ctx, sampler, speculator
        self._adapter = adapter
        self._max: Optional[int] = None
        self._stop: set = set()
        self._constraints: list = []
        self._generated: List[int] = []
        self._done = False
        self._pending: Optional[List[int]] = None   # tokens sampled but not yet fed back
        self._probes_each: List[tuple] = []
        tok = ctx.model._entry.tokenizer
        if tok is not None:
            self._stop.update(getattr(tok, "eos_tokens", []))

    def max_tokens(self, n: int) -> "Generator":
        self._max = n
        return self

    def stop(self, tokens: Iterable[int]) -> "Generator":
        self._stop = set(int(t) for t in tokens)
        return self

    def add_stop(self, tokens: Iterable[int]) -> "Generator":
        self._stop.update(int(t) for t in tokens)
        return self

    def constrain(self, c) -> "Generator":
        if hasattr(c, "build_constraint"):
            c = c.build_constraint(self.ctx.model)
        self._constraints.append(c)
        return self

    def adapter(self, a) -> "Generator":
        self._adapter = a
        return self

    def disable_system_speculation(self) -> "Generator":
        return self

    def horizon(self, n: int) -> "Generator":
        return self

    @property
    def tokens_generated(self) -> int:
        return len(self._generated)

    def is_done(self) -> bool:
        return self._done

    def __aiter__(self):
        return self

    async def __anext__(self) -> GenStep:
        if self._done or (self._max is not None and len(self._generated) >= self._max):
            self._done = True
            raise StopAsyncIteration
        ctx = self.ctx
        if self._pending is None:
            if ctx.__dict__.get("_bidir_spans"):
                await ctx._flush_media_spans()
            toks, ctx._buffer = ctx._buffer, []
            if not toks:
                raise RuntimeError("generate() needs at least one pending token in the context")
        else:
            toks = self._pending
        fwd = Forward(ctx).input(toks)
        if self._adapter is not None:
            fwd.adapter(self._adapter)
        n_draft = 0
        if self.speculator is not None and self._pending is not None:
            d_tokens, d_pos = self.speculator.draft()
            if d_tokens:
                fwd.speculative(d_tokens, d_pos or None)
                n_draft = len(d_tokens)
        last = len(toks) - 1
        if n_draft == 0 and not self._constraints and self._max is not None:
            fwd._spec_budget = max(0, self._max - len(self._generated) - 1)     # extra tokens this step may deliver
        elif n_draft == 0 and not self._constraints:
            fwd._spec_budget = 1 << 20
        handle = fwd.sample(list(range(last, last + 1 + n_draft)), self.sampler)
        for c in self._constraints:
            fwd.mask(c.step([]))
        if self._constraints or n_draft:
            fwd.pass_speculation(False)
        return GenStep(self, fwd, handle, n_draft)

    def accept(self, tokens: List[int]) -> List[int]:
        out = []
        for t in tokens:
            if self._max is not None and len(self._generated) >= self._max:
                break
            self._generated.append(t)
            out.append(t)
            for c in self._constraints:
                c.accept([t])
            if t in self._stop or any(getattr(c, "is_terminated", lambda: False)() for c in self._constraints):
                self._done = True
                break
        if self.speculator is not None:
            self.speculator.accept(out)
        if self._max is not None and len(self._generated) >= self._max:
            self._done = True
        # a run of accepted drafts already has KV for all but its last token
        self._pending = out[-1:] if out else None
        if self._done:
            # the last sampled token has no KV yet: it stays pending in the context, as after a
            # runtime-driven loop, so that a later fill or generate continues from the full text
            if self._pending:
                self.ctx._buffer.extend(self._pending)
            self._pending = None
        return out

    def _offloadable(self) -> bool:
        """Plain generation (token sampler, no constraints, no inferlet-side speculator, nothing
        generated yet) can run inside the runtime's decode cohort instead of stepping here."""
        return (not self._constraints and self.speculator is None and self._pending is None and self._adapter is None
                and not self._done and self.sampler.spec.is_token and bool(self.ctx._buffer)
                and self.ctx._entry.inference.cohorts)

    async def run_offloaded(self, on_tokens=None):
        """Hand the whole decode loop to the runtime; returns the cohort Stream when it ended."""
        ctx = self.ctx
        if ctx.__dict__.get("_bidir_spans"):
            await ctx._flush_media_spans()
        toks, ctx._buffer = ctx._buffer, []
        n = self._max if self._max is not None else 1 << 30
        start = ctx.seq_len
        await ctx._reserve_async(len(toks) + 1)
        if ctx.__dict__.get("_pending_media"):
            await ctx._await_media()
        stream = ctx._entry.inference.start_stream(ctx.id, toks, list(range(start, start + len(toks))),
                                                   self.sampler.spec, n, self._stop)
        if on_tokens is not None:
            stream.listeners.append(on_tokens)
        try:
            await host.wait(stream.done)
        except asyncio.CancelledError:
            stream.cancel()
            raise
        kept = getattr(stream, "kept", 0)
        ctx._seq_len += len(toks) + kept
        ctx._next_pos = start + len(toks) + kept
        ctx._buffer = list(stream.tokens[kept:])
        ctxm = ctx._entry.ctxm
        full = ctxm.working_page_token_count(ctx.id) // ctx.page_size
        if full:
            try:
                ctxm.commit_working_pages(ctx.id, full)
            except Exception:
                pass
        self._generated = list(stream.tokens)
        self._done = True
        return stream

    async def collect_tokens(self) -> List[int]:
        if self._offloadable():
            await self.run_offloaded()
            return list(self._generated)
        async for step in self:
            await step.execute()
        return [t for t in self._generated]

    async def collect_text(self) -> str:
        toks = await self.collect_tokens()
        stop = self._stop
        while toks and toks[-1] in stop:
            toks = toks[:-1]
        return self.ctx.model.tokenizer().decode(toks)

    async def collect_json(self, schema=None, parse=None) -> Any:
        """Constrain the output to JSON (to `schema` when given), drain, parse."""
        from .grammar import AnyJson, JsonSchema
        if not self._constraints:
            self.constrain(JsonSchema(schema) if schema is not None else AnyJson())
        value = json.loads(await self.collect_text())
        return parse(value) if parse is not None else value
