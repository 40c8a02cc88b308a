"""Samplers and probes an inferlet attaches to a forward pass (WIT `inference.sampler`).

Token samplers: argmax, multinomial, top-k, top-p, min-p, top-k+top-p. Probes: Logits,
Distribution, Logprob, Logprobs, Entropy (computed from the unscaled distribution).
Surface mirrors sdk/python/src/inferlet/sample.py:43-176.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable

from ..driver.schema import SamplerKind, SamplerSpec


class Sampler:
    def __init__(self, spec: SamplerSpec):
        self.spec = spec

    @classmethod
    def argmax(cls) -> "Sampler":
        return cls(SamplerSpec(SamplerKind.MULTINOMIAL, temperature=0.0))

    @classmethod
    def multinomial(cls, temperature: float = 1.0, seed: int = 0) -> "Sampler":
        return cls(SamplerSpec(SamplerKind.MULTINOMIAL, temperature=temperature, seed=seed))

    @classmethod
    def top_k(cls, temperature: float = 0.6, k: int = 40, seed: int = 0) -> "Sampler":
        return cls(SamplerSpec(SamplerKind.TOP_K, temperature=temperature, top_k=k, seed=seed))

    @classmethod
    def top_p(cls, temperature: float = 0.6, p: float = 0.95, seed: int = 0) -> "Sampler":
        return cls(SamplerSpec(SamplerKind.TOP_P, temperature=temperature, top_p=p, seed=seed))

    @classmethod
    def min_p(cls, temperature: float = 0.6, p: float = 0.1, seed: int = 0) -> "Sampler":
        return cls(SamplerSpec(SamplerKind.MIN_P, temperature=temperature, min_p=p, seed=seed))

    @classmethod
    def top_k_top_p(cls, temperature: float = 0.6, k: int = 40, p: float = 0.95, seed: int = 0) -> "Sampler":
        return cls(SamplerSpec(SamplerKind.TOP_K_TOP_P, temperature=temperature, top_k=k, top_p=p, seed=seed))

    @property
    def is_argmax(self) -> bool:
        return self.spec.is_token and self.spec.temperature <= 0

    def __repr__(self) -> str:
        s = self.spec
        return f"Sampler({s.kind.name.lower()}, T={s.temperature}, k={s.top_k}, p={s.top_p}, min_p={s.min_p})"


class Logits:
    """Raw pre-softmax logits of a position (f32 bytes, vocab_size * 4)."""
    spec = SamplerSpec(SamplerKind.RAW_LOGITS)


@dataclass
class Distribution:
    """Top-k token ids with their temperature-scaled probabilities."""
    temperature: float = 1.0
    k: int = 32

    @property
    def spec(self):
        return SamplerSpec(SamplerKind.DIST, temperature=self.temperature, top_k=self.k)


@dataclass
class Logprob:
    token: int

    @property
    def spec(self):
        return SamplerSpec(SamplerKind.LOGPROB, labels=(self.token,))


class Logprobs:
    def __init__(self, tokens: Iterable[int] = ()):
        self.tokens = tuple(tokens)

    @property
    def spec(self):
        return SamplerSpec(SamplerKind.LOGPROBS, labels=self.tokens)


class Entropy:
    spec = SamplerSpec(SamplerKind.ENTROPY)
