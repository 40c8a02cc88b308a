"""The host side of the inferlet contract, function by function.

`pie_b200/wit/**` states the contract in WIT (the interface names, function names and signatures of
pie-project/pie v0.4.0). This module is its native implementation: one class per WIT interface,
named `INTERFACES["<package>/<interface>"]`, with one attribute per function (kebab-case ->
snake_case), one nested class per resource and one method per resource function, taking the same
number of parameters. `result<T, error>` becomes "return T or raise WitError", `option<T>` becomes
"T or None", a `borrow<r>` parameter is the Python object of resource r. The high-level SDK
(`pie_b200.sdk.core`) and a wasm linker would both sit on exactly this surface; the reference
binds the same functions with `wasmtime::component::bindgen!` (runtime/src/api.rs:43-129, one file
per interface under runtime/src/api/). tests/test_wit_contract.py parses the WIT files and checks
every function here against them.
"""
from __future__ import annotations

import asyncio
import json as _json
from typing import Any, List, Optional, Sequence, Tuple

from ..driver.schema import SamplerKind, SamplerSpec
from . import host


class WitError(RuntimeError):
    """The `error` arm of a WIT `result`."""


def _guard(fn, *a, **kw):
    try:
        return fn(*a, **kw)
    except WitError:
        raise
    except Exception as e:  # noqa: BLE001 - the contract's error type is a string
        raise WitError(str(e)) from e


class Pollable:
    """wasi:io/poll pollable over a runtime future, an asyncio future or a plain callable."""

    def __init__(self, is_ready, waiter=None):
        self._ready, self._waiter = is_ready, waiter

    def ready(self) -> bool:
        return bool(self._ready())

    async def block(self) -> None:
        if self._waiter is not None:
            await self._waiter()
        else:
            while not self.ready():
                await asyncio.sleep(0.001)


class _FutureValue:
    """future-string / future-blob: a value that an asyncio task will deliver."""

    def __init__(self, coro):
        self._task = asyncio.ensure_future(coro)

    def pollable(self) -> Pollable:
        async def wait():
            await asyncio.wait([self._task])
        return Pollable(self._task.done, wait)

    def get(self):
        if not self._task.done():
            return None
        return self._task.result()


# ----------------------------------------------------------------------------- pie:core/types
class types:
    error = str
    blob = bytes

    class future_string(_FutureValue):
        pass

    class future_blob(_FutureValue):
        pass


# ----------------------------------------------------------------------------- pie:core/model
class model:
    class model:
        def __init__(self, sdk_model):
            self._m = sdk_model

        @staticmethod
        def load(name: str) -> "model.model":
            from .core import Model
            return model.model(_guard(Model.load, name))

        def tokenizer(self) -> "model.tokenizer":
            return model.tokenizer(self._m.tokenizer())

        def default_system_speculation(self) -> bool:
            return bool(self._m.default_system_speculation())

    class tokenizer:
        def __init__(self, sdk_tok):
            self._t = sdk_tok

        def encode(self, text: str) -> List[int]:
            return self._t.encode(text)

        def decode(self, tokens: Sequence[int]) -> str:
            return _guard(self._t.decode, tokens)

        def vocabs(self) -> Tuple[List[int], List[bytes]]:
            return self._t.vocabs()

        def split_regex(self) -> str:
            return self._t.split_regex()

        def special_tokens(self) -> Tuple[List[int], List[bytes]]:
            return self._t.special_tokens()


# ----------------------------------------------------------------------------- pie:core/context
class context:
    page_id = int

    class context:
        """A KV context at the level of the contract: explicit page reserve / commit, no token buffer."""

        def __init__(self, mdl: "model.model", cid: int):
            self._model, self._entry, self.id = mdl, mdl._m._entry, cid

        @staticmethod
        def create(mdl: "model.model") -> "context.context":
            return context.context(mdl, _guard(mdl._m._entry.ctxm.create, host.proc().id))

        @staticmethod
        def open(mdl: "model.model", name: str) -> "context.context":
            p = host.proc()
            return context.context(mdl, _guard(mdl._m._entry.ctxm.open, p.username, name, p.id))

        @staticmethod
        def take(mdl: "model.model", name: str) -> "context.context":
            p = host.proc()
            return context.context(mdl, _guard(mdl._m._entry.ctxm.take, p.username, name, p.id))

        @staticmethod
        def delete(mdl: "model.model", name: str) -> None:
            _guard(mdl._m._entry.ctxm.delete_snapshot, host.proc().username, name)

        def fork(self) -> "context.context":
            return context.context(self._model, _guard(self._entry.ctxm.fork, self.id))

        def save(self, name: str) -> None:
            _guard(self._entry.ctxm.save, self.id, host.proc().username, name)

        def snapshot(self) -> str:
            return _guard(self._entry.ctxm.snapshot, self.id, host.proc().username)

        def destroy(self) -> None:
            self._entry.inference.drop_context(self.id)
            self._entry.ctxm.destroy(self.id)

        def tokens_per_page(self) -> int:
            return self._entry.page_size

        def model(self) -> "model.model":
            return self._model

        def committed_page_count(self) -> int:
            return self._entry.ctxm.committed_page_count(self.id)

        def working_page_count(self) -> int:
            return self._entry.ctxm.working_page_count(self.id)

        def commit_working_pages(self, num_pages: int) -> None:
            _guard(self._entry.ctxm.commit_working_pages, self.id, num_pages)

        def reserve_working_pages(self, num_pages: int) -> None:
            _guard(self._entry.ctxm.reserve_working_pages, self.id, num_pages)

        def release_working_pages(self, num_pages: int) -> None:
            self._entry.ctxm.release_working_pages(self.id, num_pages)

        def working_page_token_count(self) -> int:
            return self._entry.ctxm.working_page_token_count(self.id)

        def truncate_working_page_tokens(self, num_tokens: int) -> None:
            self._entry.inference.drop_context(self.id)
            self._entry.ctxm.truncate_working_page_tokens(self.id, num_tokens)

        def suspend(self) -> None:
            self._entry.inference.drop_context(self.id)
            _guard(self._entry.ctxm.suspend, self.id)

        def bid(self, value: float) -> None:
            self._entry.ctxm.set_bid(self.id, value)


# ----------------------------------------------------------------------------- pie:core/inference
def _sampler_spec(s) -> SamplerSpec:
    """A WIT `sampler` variant as (case, payload) -> SamplerSpec. The u32 of `multinomial` is the seed."""
    if isinstance(s, SamplerSpec):
        return s
    case, payload = (s, None) if isinstance(s, str) else (s[0], s[1] if len(s) > 1 else None)
    case = case.replace("-", "_")
    if case == "multinomial":
        return SamplerSpec(SamplerKind.MULTINOMIAL, float(payload[0]), seed=int(payload[1]))
    if case == "top_k":
        return SamplerSpec(SamplerKind.TOP_K, float(payload[0]), top_k=int(payload[1]))
    if case == "top_p":
        return SamplerSpec(SamplerKind.TOP_P, float(payload[0]), top_p=float(payload[1]))
    if case == "min_p":
        return SamplerSpec(SamplerKind.MIN_P, float(payload[0]), min_p=float(payload[1]))
    if case == "top_k_top_p":
        return SamplerSpec(SamplerKind.TOP_K_TOP_P, float(payload[0]), top_k=int(payload[1]), top_p=float(payload[2]))
    if case == "embedding":
        return SamplerSpec(SamplerKind.EMBEDDING)
    if case == "dist":
        return SamplerSpec(SamplerKind.DIST, float(payload[0]), top_k=int(payload[1]))
    if case == "raw_logits":
        return SamplerSpec(SamplerKind.RAW_LOGITS)
    if case == "logprob":
        return SamplerSpec(SamplerKind.LOGPROB, labels=(int(payload),))
    if case == "logprobs":
        return SamplerSpec(SamplerKind.LOGPROBS, labels=tuple(int(t) for t in payload))
    if case == "entropy":
        return SamplerSpec(SamplerKind.ENTROPY)
    raise WitError(f"unknown sampler case {case!r}")


def _slot_output(s) -> tuple:
    """Runtime SlotOutput -> WIT `slot-output` variant as (case, payload)."""
    k = s.kind
    if k == "token":
        return ("token", int(s.token))
    if k == "distribution":
        return ("distribution", (list(s.ids), list(s.probs)))
    if k == "logits":
        return ("logits", bytes(s.logits))
    if k == "logprobs":
        return ("logprobs", list(s.logprobs))
    if k == "entropy":
        return ("entropy", float(s.entropy))
    return ("embedding", bytes(s.logits or b""))


class inference:
    brle = list

    class forward_pass:
        def __init__(self, mdl: "model.model"):
            self._model = mdl
            self._ctx: Optional[context.context] = None
            self._tokens: List[int] = []
            self._positions: List[int] = []
            self._spec_tokens: List[int] = []
            self._spec_positions: List[int] = []
            self._samplers: List[tuple] = []
            self._attn: Optional[List[List[int]]] = None
            self._mask: Optional[List[int]] = None
            self._adapter = -1
            self._pass_spec = True
            self._system_spec = mdl.default_system_speculation()
            self._media: List[tuple] = []
            self._adapter_seed: Optional[int] = None

        def context(self, ctx: "context.context") -> None:
            self._ctx = ctx

        def input_tokens(self, tokens: Sequence[int], positions: Sequence[int]) -> None:
            self._tokens.extend(int(t) for t in tokens)
            self._positions.extend(int(p) for p in positions)

        def input_image(self, image: "media.image", anchor: int) -> None:
            self._media.append(("image", image, int(anchor)))

        def input_audio(self, audio: "media.audio", anchor: int) -> None:
            self._media.append(("audio", audio, int(anchor)))

        def input_speculative_tokens(self, tokens: Sequence[int], positions: Sequence[int]) -> None:
            self._spec_tokens = [int(t) for t in tokens]
            self._spec_positions = [int(p) for p in positions]

        def output_speculative_tokens(self, flag: bool) -> None:
            self._system_spec = bool(flag)

        def pass_speculation(self, flag: bool) -> None:
            self._pass_spec = bool(flag)

        def attention_mask(self, mask: Sequence[Sequence[int]]) -> None:
            self._attn = [list(m) for m in mask]

        def logit_mask(self, mask: Sequence[int]) -> None:
            self._mask = list(mask)

        def sampler(self, indices: Sequence[int], sampler) -> None:
            spec = _sampler_spec(sampler)
            self._samplers.append(([int(i) for i in indices], spec))

        def adapter(self, adapter: "adapter.adapter") -> None:
            self._adapter = adapter.id

        def execute(self) -> "inference.future_output":
            if self._ctx is None:
                raise WitError("forward-pass.execute: no context attached")
            waits = []
            if self._media:
                # a spliced clip: the driver encodes it (once per distinct content) and the rows of this pass at positions
                # anchor .. anchor + token-count take the encoder's rows instead of their tokens' embeddings
                entry = self._ctx._entry
                kinds = getattr(entry.caps[0], "media", ()) or ()
                for kind, clip, anchor in self._media:
                    if kind not in kinds or entry.media is None:
                        raise WitError(f"model has no {kind} encoder")
                    rows = clip.token_count()
                    try:
                        at = self._positions.index(anchor)
                    except ValueError:
                        raise WitError(f"input-{kind}: no input token at position {anchor}") from None
                    if self._positions[at:at + rows] != list(range(anchor, anchor + rows)):
                        raise WitError(f"input-{kind}: the pass must carry {rows} consecutive positions from {anchor} for the clip")
                    toks, e = _guard(entry.media.put, self._ctx.id, kind, clip._array(), clip._grids(), rows)
                    self._tokens[at:at + rows] = toks
                    if not e.ready.done():
                        waits.append(e.ready)
            flat = [(i, spec) for idx, spec in self._samplers for i in idx]
            groups = [len(idx) for idx, _ in self._samplers]
            svc = self._ctx._entry.inference
            args = (self._ctx.id, self._tokens, self._positions, flat, self._attn, self._mask,
                    self._spec_tokens, self._spec_positions, self._adapter, self._pass_spec)
            if not waits:
                return inference.future_output(_guard(svc.submit, *args), groups)
            # the pass goes to the scheduler once every encoder has finished; an encoder's error is the pass's error
            from ..runtime.inference import Future
            out, left, loop = Future(), [len(waits)], asyncio.get_running_loop()

            def go():
                try:
                    svc.submit(*args).add_done_callback(lambda g: out.set(g._result, g._exc))
                except Exception as exc:  # noqa: BLE001
                    out.set(None, exc)

            def ready(f):
                if f._exc is not None:
                    out.set(None, f._exc)
                    return
                left[0] -= 1
                if left[0] == 0:
                    loop.call_soon_threadsafe(go)
            for f in waits:
                f.add_done_callback(ready)
            return inference.future_output(out, groups)

    class future_output:
        def __init__(self, fut, groups: List[int]):
            self._fut, self._groups = fut, groups

        def pollable(self) -> Pollable:
            async def wait():
                try:
                    await host.wait(self._fut)
                except Exception:  # noqa: BLE001 - get() reports it
                    pass
            return Pollable(self._fut.done, wait)

        def get(self) -> Optional[dict]:
            if not self._fut.done():
                return None
            raw = _guard(self._fut.result)
            slots = [_slot_output(s) for s in raw.slots]
            return {"slots": slots, "spec_tokens": list(getattr(raw, "spec_tokens", []) or []),
                    "spec_positions": list(getattr(raw, "spec_positions", []) or [])}

    class grammar:
        def __init__(self, g):
            self._g = g

        @staticmethod
        def from_json_schema(schema: str) -> "inference.grammar":
            from ..runtime.structured import Grammar
            return inference.grammar(_guard(Grammar.from_json_schema, schema))

        @staticmethod
        def json() -> "inference.grammar":
            from ..runtime.structured import Grammar
            return inference.grammar(Grammar.json())

        @staticmethod
        def from_regex(pattern: str) -> "inference.grammar":
            from ..runtime.structured import Grammar
            return inference.grammar(_guard(Grammar.from_regex, pattern))

        @staticmethod
        def from_ebnf(ebnf: str) -> "inference.grammar":
            from ..runtime.structured import Grammar
            return inference.grammar(_guard(Grammar.from_ebnf, ebnf))

        def to_string(self) -> str:
            return self._g.to_string()

    class matcher:
        def __init__(self, grammar: "inference.grammar", tokenizer: "model.tokenizer"):
            from ..runtime.structured import Matcher
            self._m = _guard(Matcher, grammar._g, tokenizer._t._t)

        def accept_tokens(self, token_ids: Sequence[int]) -> None:
            _guard(self._m.accept_tokens, [int(t) for t in token_ids])

        def next_token_logit_mask(self) -> List[int]:
            return list(self._m.next_token_logit_mask())

        def is_terminated(self) -> bool:
            return bool(self._m.is_terminated())

        def reset(self) -> None:
            self._m.reset()


# ----------------------------------------------------------------------------- pie:core/runtime
class runtime:
    @staticmethod
    def version() -> str:
        from . import runtime as rt
        return rt.version()

    @staticmethod
    def instance_id() -> str:
        return host.proc().id

    @staticmethod
    def username() -> str:
        return host.proc().username

    @staticmethod
    def models() -> List[str]:
        from . import runtime as rt
        return rt.models()

    @staticmethod
    def launch(program: str, input: str) -> "runtime.child":  # noqa: A002 - the contract's parameter name
        from . import runtime as rt
        try:
            arg = _json.loads(input) if input else None
        except ValueError:
            arg = input
        return runtime.child(_guard(rt.launch, program, arg))

    class child:
        def __init__(self, sdk_child):
            self._c = sdk_child

        def pollable(self) -> Pollable:
            return Pollable(lambda: self._c.get() is not None or self._c._proc.done.is_set())

        def get(self):
            """option<result<string, error>>: None while running, then ("ok", value) or ("err", message)."""
            if not self._c._proc.done.is_set():
                return None
            try:
                return ("ok", self._c.get())
            except Exception as e:  # noqa: BLE001
                return ("err", str(e))

        def pid(self) -> str:
            return self._c.pid

        def cancel(self) -> None:
            self._c.cancel()


# ----------------------------------------------------------------------------- pie:core/scheduling
class scheduling:
    @staticmethod
    def price() -> float:
        from . import scheduling as sc
        return sc.price()

    @staticmethod
    def rent(ctx: "context.context") -> float:
        from . import scheduling as sc
        return float(sc.rent(ctx))

    @staticmethod
    def dividend(model: "model.model") -> float:  # noqa: A002
        from . import scheduling as sc
        return float(sc.dividend(model._m))

    @staticmethod
    def latency(ctx: "context.context") -> float:
        from . import scheduling as sc
        return float(sc.latency(ctx))

    @staticmethod
    def balance(model: "model.model") -> float:  # noqa: A002
        from . import scheduling as sc
        return float(sc.balance(model._m))


# ----------------------------------------------------------------------------- pie:core/session
class session:
    @staticmethod
    def send(message: str) -> None:
        from . import session as ss
        ss.send(message)

    @staticmethod
    def receive() -> "types.future_string":
        from . import session as ss
        return types.future_string(ss.receive())

    @staticmethod
    def send_file(data: bytes) -> None:
        from . import session as ss
        ss.send_file(data)

    @staticmethod
    def receive_file() -> "types.future_blob":
        from . import session as ss
        return types.future_blob(ss.receive_file())


# ----------------------------------------------------------------------------- pie:core/messaging
class messaging:
    class subscription:
        def __init__(self, sub):
            self._s = sub

        def pollable(self) -> Pollable:
            return Pollable(lambda: not self._s.queue.empty() if hasattr(self._s, "queue") else True)

        def get(self) -> Optional[str]:
            q = getattr(self._s, "queue", None)
            if q is None or q.empty():
                return None
            return q.get_nowait()

        def unsubscribe(self) -> None:
            self._s.unsubscribe()

    @staticmethod
    def push(topic: str, message: str) -> None:
        host.engine().messaging.push(topic, message)

    @staticmethod
    def pull(topic: str) -> "types.future_string":
        return types.future_string(host.engine().messaging.pull(topic))

    @staticmethod
    def broadcast(topic: str, message: str) -> None:
        host.engine().messaging.broadcast(topic, message)

    @staticmethod
    def subscribe(topic: str) -> "messaging.subscription":
        return messaging.subscription(host.engine().messaging.subscribe(topic))


# ----------------------------------------------------------------------------- pie:core/adapter
class adapter:
    class adapter:
        """Adapters are named: `create` registers a fresh one under `name`, `open` finds it again."""
        _names: dict = {}

        def __init__(self, mdl: "model.model", aid: int, name: str):
            self._model, self.id, self.name = mdl, aid, name

        @staticmethod
        def _svc(mdl):
            return mdl._m._entry.adapters

        @staticmethod
        def create(mdl: "model.model", name: str) -> "adapter.adapter":
            aid = _guard(adapter.adapter._svc(mdl).create, host.proc().id, 8, 16.0, 0)
            adapter.adapter._names[(mdl._m.name, name)] = aid
            return adapter.adapter(mdl, aid, name)

        def destroy(self) -> None:
            self._svc(self._model).destroy(self.id)
            self._names.pop((self._model._m.name, self.name), None)

        @staticmethod
        def open(mdl: "model.model", name: str) -> Optional["adapter.adapter"]:
            aid = adapter.adapter._names.get((mdl._m.name, name))
            if aid is None:
                try:
                    aid = adapter.adapter._svc(mdl).load(host.proc().id, name)
                except Exception:  # noqa: BLE001 - option<adapter>
                    return None
            return adapter.adapter(mdl, aid, name)

        def fork(self, name: str) -> "adapter.adapter":
            aid = self._svc(self._model).fork(self.id, host.proc().id)
            self._names[(self._model._m.name, name)] = aid
            return adapter.adapter(self._model, aid, name)

        def load(self, path: str) -> None:
            """Replace this adapter's weights with those stored under `path` (a name in the adapter store)."""
            svc = self._svc(self._model)
            new = _guard(svc.load, host.proc().id, path)
            svc.destroy(self.id)
            self.id = new
            self._names[(self._model._m.name, self.name)] = new

        def save(self, path: str) -> None:
            _guard(self._svc(self._model).save, self.id, path)


# ----------------------------------------------------------------------------- pie:core/media
def _marker_tokens(mdl, kind: str, side: int) -> List[int]:
    """The model's own span marker before (0) or after (1) a clip of `kind`, tokenised; [] where it has none."""
    if mdl is None:
        return []
    spec = getattr(mdl._m._entry.caps[0], "media_spec", None) or {}
    text = ((spec.get("delimiters") or {}).get(kind) or ("", ""))[side]
    return list(mdl._m.tokenizer().encode(text)) if text else []


class media:
    class image:
        def __init__(self, feats, mdl=None):
            self._f, self._mdl = feats, mdl

        @staticmethod
        def from_bytes(mdl: "model.model", bytes: bytes) -> "media.image":  # noqa: A002
            from . import media as md
            return media.image(_guard(md.Image.for_model, mdl._m, bytes).features, mdl)

        def token_count(self) -> int:
            return int(self._f.num_tokens)

        def position_span(self) -> int:
            """Positions the clip advances the sequence by: its rows (the language models here use one-dimensional
            positions for image rows)."""
            return self.token_count()

        def grid(self) -> Tuple[int, int, int]:
            g = self._f.grid
            return (int(g[0]), int(g[1]), int(g[2]))

        def prefix_tokens(self) -> List[int]:
            return _marker_tokens(self._mdl, "image", 0)

        def suffix_tokens(self) -> List[int]:
            return _marker_tokens(self._mdl, "image", 1)

        def _array(self):
            return self._f.patches

        def _grids(self):
            return [self._f.grid]

    class video:
        def __init__(self, mdl, frames):
            self._m, self._frames = mdl, frames

        @staticmethod
        def from_bytes(mdl: "model.model", bytes: bytes, max_frames: int) -> "media.video":  # noqa: A002
            from ..runtime import multimodal as mm
            return media.video(mdl, _guard(mm.decode_frames, bytes, max_frames))

        def frame_count(self) -> int:
            return len(self._frames)

        def frame(self, index: int) -> "media.image":
            from . import media as md
            if not 0 <= index < len(self._frames):
                raise WitError("frame index out of range")
            return media.image(md._features_for(self._m._m, [self._frames[index]], {}), self._m)

        def timestamp(self, index: int) -> float:
            return float(index)

    class audio:
        def __init__(self, mel, mdl=None):
            self._mel, self._mdl = mel, mdl

        @staticmethod
        def from_bytes(mdl: "model.model", bytes: bytes) -> "media.audio":  # noqa: A002
            from ..runtime import multimodal as mm
            return media.audio(_guard(mm.audio_features, bytes), mdl)

        def token_count(self) -> int:
            f = int(self._mel.shape[1])
            return ((f - 1) // 2 + 1) // 2 if f > 0 else 0       # a stride-2 convolution, then a stride-2 pool: one row per 40 ms

        def position_span(self) -> int:
            return self.token_count()

        def prefix_tokens(self) -> List[int]:
            return _marker_tokens(self._mdl, "audio", 0)

        def suffix_tokens(self) -> List[int]:
            return _marker_tokens(self._mdl, "audio", 1)

        def _array(self):
            return self._mel

        def _grids(self):
            return [(int(self._mel.shape[1]),)]


# ----------------------------------------------------------------------------- pie:core/audio-out
class audio_out:
    class speech:
        """Speech synthesis needs a model with an audio decoder; the text-only families have none."""

        def __init__(self, pcm, rate: int):
            self._pcm, self._rate = pcm, rate

        @staticmethod
        def generate(mdl: "model.model", req: dict) -> "audio_out.speech":
            kinds = getattr(mdl._m._entry.caps[0], "media", ()) or ()
            if "audio-out" not in kinds:
                raise WitError(f"model {mdl._m.name} has no audio decoder")
            drv = mdl._m._entry.drivers[0]
            pcm, rate = _guard(drv.generate_audio, req)
            return audio_out.speech(pcm, rate)

        def sample_rate(self) -> int:
            return self._rate

        def channels(self) -> int:
            return 1

        def duration_ms(self) -> int:
            return int(1000 * len(self._pcm) / max(1, self._rate))

        def pcm(self) -> List[float]:
            return [float(x) for x in self._pcm]


# ----------------------------------------------------------------------------- pie:instruct/*
def _instruct(mdl: "model.model"):
    ins = mdl._m.instruct
    if ins is None:
        raise WitError(f"model {mdl._m.name} has no chat template")
    return ins


def _raw_tok(mdl: "model.model"):
    return mdl._m.tokenizer()


class _TextDecoder:
    """decoder resources of pie:instruct: tokens in, one event out (the last event of the chunk)."""

    def __init__(self, mdl: "model.model", impl, text_input: bool):
        self._tok, self._d, self._text = _raw_tok(mdl), impl, text_input

    def _event(self, ev) -> tuple:
        raise NotImplementedError

    def feed(self, tokens: Sequence[int]) -> tuple:
        try:
            evs = self._d.feed(self._tok.decode(list(tokens)) if self._text else list(tokens))
        except Exception as e:  # noqa: BLE001
            raise WitError(str(e)) from e
        return self._event(evs[-1] if evs else None)

    def reset(self) -> None:
        if hasattr(self._d, "reset"):
            self._d.reset()


class chat:
    @staticmethod
    def system(model: "model.model", message: str) -> List[int]:  # noqa: A002
        return _instruct(model).render("system", message, _raw_tok(model), first=True)

    @staticmethod
    def user(model: "model.model", message: str) -> List[int]:  # noqa: A002
        return _instruct(model).render("user", message, _raw_tok(model))

    @staticmethod
    def assistant(model: "model.model", message: str) -> List[int]:  # noqa: A002
        return _instruct(model).render("assistant", message, _raw_tok(model))

    @staticmethod
    def cue(model: "model.model") -> List[int]:  # noqa: A002
        return _instruct(model).cue(_raw_tok(model))

    @staticmethod
    def seal(model: "model.model") -> List[int]:  # noqa: A002
        return _instruct(model).seal(_raw_tok(model))

    @staticmethod
    def stop_tokens(model: "model.model") -> List[int]:  # noqa: A002
        return list(_instruct(model).stop_tokens(_raw_tok(model)))

    @staticmethod
    def create_decoder(model: "model.model") -> "chat.decoder":  # noqa: A002
        return chat.decoder(model)

    class decoder(_TextDecoder):
        def __init__(self, mdl: "model.model"):
            from ..runtime.instruct import ChatDecoder
            super().__init__(mdl, ChatDecoder(_raw_tok(mdl)._t, _instruct(mdl)), text_input=False)

        def _event(self, ev) -> tuple:
            if ev is None:
                return ("delta", "")
            if ev.kind == "done":
                return ("done", getattr(ev, "text", ""))
            if ev.kind == "interrupt":
                return ("interrupt", int(getattr(ev, "token", 0)))
            return ("delta", getattr(ev, "text", ""))


class reasoning:
    @staticmethod
    def create_decoder(model: "model.model") -> "reasoning.decoder":  # noqa: A002
        return reasoning.decoder(model)

    class decoder(_TextDecoder):
        def __init__(self, mdl: "model.model"):
            from ..runtime.instruct import ReasoningDecoder
            super().__init__(mdl, ReasoningDecoder(_instruct(mdl)), text_input=True)

        def _event(self, ev) -> tuple:
            if ev is None:
                return ("delta", "")
            if ev.kind in ("think_start", "start"):
                return ("start", None)
            if ev.kind in ("think_end", "complete"):
                return ("complete", getattr(ev, "text", ""))
            return ("delta", getattr(ev, "text", ""))


class tool_use:
    @staticmethod
    def _tools(tools: Sequence[str]) -> List[dict]:
        return [_json.loads(t) if isinstance(t, str) else t for t in tools]

    @staticmethod
    def equip(model: "model.model", tools: Sequence[str]) -> List[int]:  # noqa: A002
        text = _guard(_instruct(model).equip, tool_use._tools(tools))
        return _raw_tok(model).encode(text)

    @staticmethod
    def answer(model: "model.model", name: str, value: str) -> List[int]:  # noqa: A002
        return _raw_tok(model).encode(_instruct(model).answer(name, value))

    @staticmethod
    def create_decoder(model: "model.model") -> "tool_use.decoder":  # noqa: A002
        return tool_use.decoder(model)

    @staticmethod
    def format(model: "model.model", tools: Sequence[str]) -> Optional["inference.grammar"]:  # noqa: A002
        try:
            return inference.grammar.from_ebnf(_instruct(model).tool_grammar(tool_use._tools(tools)))
        except Exception:  # noqa: BLE001 - option<grammar>: a family without a tool format
            return None

    @staticmethod
    def create_matcher(model: "model.model", tools: Sequence[str]) -> "inference.matcher":  # noqa: A002
        g = tool_use.format(model, tools)
        if g is None:
            raise WitError("this model family has no tool-call format")
        return inference.matcher(g, model.tokenizer())

    class decoder(_TextDecoder):
        def __init__(self, mdl: "model.model"):
            from ..runtime.instruct import ToolDecoder
            super().__init__(mdl, ToolDecoder(_instruct(mdl)), text_input=True)

        def _event(self, ev) -> tuple:
            if ev is not None and ev.kind == "tool_call":
                call = ev.call
                return ("call", (call.get("name", ""), _json.dumps(call.get("arguments", {}))))
            return ("start", None)


# ----------------------------------------------------------------------------- pie:mcp/*
class mcp_types:
    json = str

    @staticmethod
    def error(code: int, message: str, data: Optional[str] = None) -> dict:
        return {"code": int(code), "message": message, "data": data}


class mcp_client:
    class session:
        """Requests go to the client that registered the server and come back as JSON text."""

        def __init__(self, server: str):
            self._server = server

        async def _call(self, method: str, params=None) -> str:
            from . import mcp
            try:
                return _json.dumps(await mcp.request(self._server, method, params))
            except mcp.McpError as e:
                raise WitError(_json.dumps(mcp_types.error(getattr(e, "code", -32000), str(e)))) from e

        def list_tools(self):
            return self._call("tools/list")

        def call_tool(self, name: str, args: str):
            return self._call("tools/call", {"name": name, "arguments": _json.loads(args) if args else {}})

        def list_resources(self):
            return self._call("resources/list")

        def read_resource(self, uri: str):
            return self._call("resources/read", {"uri": uri})

        def list_prompts(self):
            return self._call("prompts/list")

        def get_prompt(self, name: str, args: str):
            return self._call("prompts/get", {"name": name, "arguments": _json.loads(args) if args else {}})

    @staticmethod
    def available_servers() -> List[str]:
        return sorted(getattr(host.engine(), "mcp_servers", {}) or {})

    @staticmethod
    def connect(server_name: str) -> "mcp_client.session":
        if server_name not in (getattr(host.engine(), "mcp_servers", {}) or {}):
            raise WitError(_json.dumps(mcp_types.error(-32001, f"no MCP server {server_name!r} registered")))
        return mcp_client.session(server_name)


# ----------------------------------------------------------------------------- pie:zo/zo
class zo:
    @staticmethod
    def adapter_seed(self: "inference.forward_pass", seed: int) -> None:  # noqa: N805 - the contract names it self
        self._adapter_seed = int(seed)

    @staticmethod
    def initialize(self: "adapter.adapter", rank: int, alpha: float, population_size: int, mu_fraction: float,  # noqa: N805
                   initial_sigma: float) -> None:
        svc = self._svc(self._model)
        info = svc.adapters.get(self.id)
        if info is not None and (info.rank != rank or abs(info.alpha - alpha) > 1e-9):
            new = _guard(svc.create, host.proc().id, int(rank), float(alpha), 0)
            svc.destroy(self.id)
            self.id = new
            self._names[(self._model._m.name, self.name)] = new
        self.population_size, self.mu_fraction = int(population_size), float(mu_fraction)
        _guard(svc.zo_init, self.id, float(initial_sigma))

    @staticmethod
    def update(self: "adapter.adapter", scores: Sequence[float], seeds: Sequence[int], max_sigma: float) -> None:  # noqa: N805
        svc = self._svc(self._model)
        info = svc.adapters.get(self.id)
        if info is not None and max_sigma > 0:
            info.zo_sigma = min(info.zo_sigma, float(max_sigma))
        _guard(svc.zo_update, self.id, [int(s) for s in seeds], [float(x) for x in scores], 1e-2)


INTERFACES = {
    "pie:core/types": types, "pie:core/model": model, "pie:core/context": context, "pie:core/inference": inference,
    "pie:core/runtime": runtime, "pie:core/scheduling": scheduling, "pie:core/session": session,
    "pie:core/messaging": messaging, "pie:core/adapter": adapter, "pie:core/media": media,
    "pie:core/audio-out": audio_out, "pie:instruct/chat": chat, "pie:instruct/reasoning": reasoning,
    "pie:instruct/tool-use": tool_use, "pie:mcp/types": mcp_types, "pie:mcp/client": mcp_client, "pie:zo/zo": zo,
}
