"""LoRA adapters for inferlets (WIT `pie:core/adapter` and `pie:zo`).

    ad = Adapter.create(model, rank=8, alpha=16)       # or Adapter.load(model, "my-adapter")
    out = await ctx.forward().input(tokens).adapter(ad).sample([...], sampler).execute()
    gen = ctx.generate(sampler, max_tokens=32, adapter=ad)
    ad.save("my-adapter"); ad.destroy()

Counterpart of sdk/python/src/inferlet/adapter.py and zo.py.
"""
from __future__ import annotations

from typing import List

from . import host


class Adapter:
    def __init__(self, model, aid: int):
        self.model, self.id = model, aid

    @staticmethod
    def _svc(model):
        return model._entry.adapters

    @classmethod
    def create(cls, model, rank: int = 8, alpha: float = 16.0, seed: int = 0) -> "Adapter":
        return cls(model, cls._svc(model).create(host.proc().id, rank, alpha, seed))

    @classmethod
    def load(cls, model, name: str) -> "Adapter":
        return cls(model, cls._svc(model).load(host.proc().id, name))

    def fork(self) -> "Adapter":
        return Adapter(self.model, self._svc(self.model).fork(self.id, host.proc().id))

    def save(self, name: str) -> None:
        self._svc(self.model).save(self.id, name)

    def destroy(self) -> None:
        self._svc(self.model).destroy(self.id)

    # ---- zeroth-order optimisation (pie:zo)
    def zo_init(self, sigma: float = 1e-3) -> None:
        self._svc(self.model).zo_init(self.id, sigma)

    def zo_perturb(self, seed: int, sign: float = 1.0) -> None:
        self._svc(self.model).zo_perturb(self.id, seed, sign)

    def zo_update(self, seeds: List[int], scores: List[float], lr: float = 1e-2) -> None:
        self._svc(self.model).zo_update(self.id, seeds, scores, lr)
