"""Drivers without a model: the dummy driver (shape-correct random outputs, for plumbing) and a
scriptable mock driver (for scheduler / KV / failure tests on a CPU).

Dummy: counterpart of the reference's dummy driver (driver/dummy/src/handler.rs: random tokens
that honour logit masks). Mock: counterpart of its test fixture
(runtime/tests/common/mock_device.rs:24-200: Echo / Counter / Delayed / FailAfter behaviours
and a call recorder).
"""
from __future__ import annotations

import threading
import time
from typing import Callable, List, Optional

import numpy as np

from ..runtime import brle
from .schema import (Capabilities, CopyRequest, ForwardRequest, ForwardResponse, SamplerKind, SlotOutput)


class Behavior:
    """Decides the token of every token-sampler slot of a batch."""

    def tokens(self, req: ForwardRequest, rows: np.ndarray) -> np.ndarray:
        raise NotImplementedError

    def before(self, req: ForwardRequest) -> None:
        pass


class EchoBehavior(Behavior):
    """Samples the input token at the sampled row (token in -> same token out)."""

    def tokens(self, req, rows):
        return np.asarray(req.tokens)[rows]


class CounterBehavior(Behavior):
    """Sampled token = input token + 1 (mod vocab): makes generation order checkable."""

    def __init__(self, vocab: int = 32000):
        self.vocab = vocab

    def tokens(self, req, rows):
        return (np.asarray(req.tokens)[rows] + 1) % self.vocab


class ScriptedBehavior(Behavior):
    """Answers the sampled rows with the next tokens of a fixed script, one per row in call order (the script's last
    token repeats when it runs out): lets a test make the "model" say a chosen reply."""

    def __init__(self, script):
        self.script, self.i = [int(t) for t in script], 0

    def tokens(self, req, rows):
        out = np.empty(len(rows), dtype=np.int64)
        for k in range(len(rows)):
            out[k] = self.script[min(self.i, len(self.script) - 1)]
            self.i += 1
        return out


class DelayedBehavior(Behavior):
    def __init__(self, inner: Behavior, seconds: float):
        self.inner, self.seconds = inner, seconds

    def before(self, req):
        time.sleep(self.seconds)

    def tokens(self, req, rows):
        return self.inner.tokens(req, rows)


class FailAfterBehavior(Behavior):
    """Succeeds `n` fires, then every fire raises (a driver that dies mid-run)."""

    def __init__(self, inner: Behavior, n: int):
        self.inner, self.n, self.count = inner, n, 0

    def before(self, req):
        self.count += 1
        if self.count > self.n:
            raise RuntimeError(f"mock driver failure after {self.n} fires")

    def tokens(self, req, rows):
        return self.inner.tokens(req, rows)


class RandomBehavior(Behavior):
    def __init__(self, vocab: int, seed: int = 0):
        self.vocab, self.rng = vocab, np.random.default_rng(seed)

    def tokens(self, req, rows):
        return self.rng.integers(0, self.vocab, len(rows))


class CallRecorder:
    def __init__(self, keep_requests: bool = False):
        self.fires: List[dict] = []
        self.copies: List[CopyRequest] = []
        self.requests: List[ForwardRequest] = []      # the requests themselves, when asked to keep them
        self.keep_requests = keep_requests
        self.lock = threading.Lock()

    def record_fire(self, req: ForwardRequest) -> None:
        with self.lock:
            if self.keep_requests:
                self.requests.append(req)
            self.fires.append({"requests": req.num_requests, "tokens": req.num_tokens,
                               "slots": len(req.slot_samplers), "page_refs": len(req.kv_page_indices),
                               "masked": bool(req.has_user_mask is not None and req.has_user_mask.any()),
                               "context_ids": None if req.context_ids is None else req.context_ids.tolist()})


class MockDriver:
    def __init__(self, behavior: Optional[Behavior] = None, total_pages: int = 64, page_size: int = 16,
                 max_requests: int = 64, max_tokens: int = 1024, vocab: int = 32000, swap_pages: int = 0,
                 recorder: Optional[CallRecorder] = None):
        self.behavior = behavior or CounterBehavior(vocab)
        self.caps = Capabilities(total_pages=total_pages, kv_page_size=page_size, max_forward_requests=max_requests,
                                 max_forward_tokens=max_tokens, vocab_size=vocab, arch_name="mock",
                                 swap_pool_size=swap_pages, max_model_len=1 << 20)
        self.recorder = recorder or CallRecorder()
        self.alive = True
        self.vocab = vocab
        self._prev_tokens = None

    def capabilities(self) -> Capabilities:
        return self.caps

    def fire_batch(self, req: ForwardRequest) -> ForwardResponse:
        if not self.alive:
            raise RuntimeError("driver is not running")
        self.behavior.before(req)
        self.recorder.record_fire(req)
        rows = np.asarray(req.slot_row, dtype=np.int64) if req.slot_row is not None else np.zeros(0, np.int64)
        toks = np.asarray(self.behavior.tokens(req, rows), dtype=np.int64) if len(rows) else np.zeros(0, np.int64)
        slots = []
        for i, sp in enumerate(req.slot_samplers):
            t = int(toks[i])
            mask = req.logit_masks[int(req.slot_req[i])] if req.logit_masks else None
            if mask is not None:
                allowed = np.flatnonzero(brle.decode(mask, self.vocab))
                if len(allowed):
                    t = int(allowed[t % len(allowed)])
            if sp.is_token:
                slots.append(SlotOutput("token", token=t))
            elif sp.kind == SamplerKind.DIST:
                k = max(1, sp.top_k or 1)
                slots.append(SlotOutput("distribution", ids=[(t + j) % self.vocab for j in range(k)],
                                        probs=[1.0 / k] * k))
            elif sp.kind == SamplerKind.RAW_LOGITS:
                slots.append(SlotOutput("logits", logits=np.zeros(self.vocab, np.float32).tobytes()))
            elif sp.kind in (SamplerKind.LOGPROB, SamplerKind.LOGPROBS):
                slots.append(SlotOutput("logprobs", logprobs=[-1.0] * max(1, len(sp.labels))))
            elif sp.kind == SamplerKind.ENTROPY:
                slots.append(SlotOutput("entropy", entropy=1.0))
            else:
                slots.append(SlotOutput("embedding", logits=b""))
        all_tok = all(s.kind == "token" for s in slots)
        resp = ForwardResponse(slots=slots, tokens=np.array([s.token for s in slots], np.int32) if all_tok else None)
        if req.spec_counts is not None and np.any(req.spec_counts):
            from .schema import verify_drafts
            resp.spec_accepted = verify_drafts(req, {int(req.slot_row[i]): s.token for i, s in enumerate(slots)
                                                     if s.kind == "token"})
        return resp

    def decode_async(self, step, parity: int):
        """Array-form decode step (the cohort path) on top of the behaviour."""
        from .executor import AsyncTokens
        toks = np.array(step.host_tokens, dtype=np.int32)
        sel = step.src_row >= 0
        if sel.any():
            toks[sel] = self._prev_tokens[step.src_row[sel]]
        r = step.r
        req = ForwardRequest(tokens=toks, positions=step.positions, qo_indptr=np.arange(r + 1, dtype=np.int32),
                             kv_page_indices=step.page_indices, kv_page_indptr=step.page_indptr,
                             kv_last_page_lens=((step.kv_lens - 1) % self.caps.kv_page_size + 1).astype(np.int32),
                             slot_req=np.arange(r, dtype=np.int32), slot_row=np.arange(r, dtype=np.int32),
                             slot_samplers=[], single_token_mode=True)
        self.behavior.before(req)
        self.recorder.record_fire(req)
        out = np.asarray(self.behavior.tokens(req, np.arange(r)), dtype=np.int32)
        self._prev_tokens = out
        return AsyncTokens(None, None, r, ready=out)

    def copy(self, req: CopyRequest) -> None:
        self.recorder.copies.append(req)

    def copy_rs(self, src_slot: int, dst_slot: int) -> None:
        self.recorder.copies.append(("rs", int(src_slot), int(dst_slot)))

    def health(self) -> bool:
        return self.alive

    def kill(self) -> None:
        self.alive = False

    def shutdown(self) -> None:
        self.alive = False


class DummyDriver(MockDriver):
    """Random tokens of the right shape; masks honoured. For plumbing runs without a model."""

    def __init__(self, vocab: int = 32000, seed: int = 0, **kw):
        super().__init__(RandomBehavior(vocab, seed), vocab=vocab, **kw)
        self.caps.arch_name = "dummy"
