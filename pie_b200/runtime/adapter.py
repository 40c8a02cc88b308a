"""Adapter service of one model: LoRA adapter ids and their lifecycle
(create / destroy / fork / load / save) plus zeroth-order initialise and update, fanned out to
every driver replica of the model. Saved adapters live under a directory as
`<name>.safetensors`. Counterpart of runtime/src/adapter.rs:1-90 and runtime/src/api/{adapter,zo}.rs.
"""
from __future__ import annotations

import itertools
import os
import re
import threading
from dataclasses import dataclass
from typing import Dict, List, Optional


class AdapterError(RuntimeError):
    pass


@dataclass
class AdapterInfo:
    id: int
    owner: str            # process id
    rank: int
    alpha: float
    name: str = ""
    zo_sigma: float = 0.0


class AdapterService:
    def __init__(self, drivers: list, directory: Optional[str] = None):
        self.drivers = drivers
        self.dir = directory
        self.adapters: Dict[int, AdapterInfo] = {}
        self._ids = itertools.count(1)
        self._lock = threading.Lock()

    def _supported(self) -> None:
        if not all(hasattr(d, "create_adapter") for d in self.drivers):
            raise AdapterError("this model's driver does not serve adapters")

    def _get(self, aid: int) -> AdapterInfo:
        if aid not in self.adapters:
            raise AdapterError(f"unknown adapter {aid}")
        return self.adapters[aid]

    def _path(self, name: str) -> str:
        if not re.fullmatch(r"[A-Za-z0-9_.-]{1,64}", name):
            raise AdapterError(f"bad adapter name {name!r}")
        if not self.dir:
            raise AdapterError("no adapter directory configured")
        os.makedirs(self.dir, exist_ok=True)
        return os.path.join(self.dir, name + ".safetensors")

    # ---- lifecycle
    def create(self, owner: str, rank: int = 8, alpha: float = 16.0, seed: int = 0) -> int:
        self._supported()
        if not 1 <= rank <= 256:
            raise AdapterError("rank must be in [1, 256]")
        with self._lock:
            aid = next(self._ids)
            for d in self.drivers:
                d.create_adapter(aid, rank, alpha, seed)
            self.adapters[aid] = AdapterInfo(aid, owner, rank, alpha)
        return aid

    def destroy(self, aid: int) -> None:
        with self._lock:
            if self.adapters.pop(aid, None) is not None:
                for d in self.drivers:
                    d.destroy_adapter(aid)

    def fork(self, aid: int, owner: str) -> int:
        src = self._get(aid)
        with self._lock:
            new = next(self._ids)
            for d in self.drivers:
                d.fork_adapter(aid, new)
            self.adapters[new] = AdapterInfo(new, owner, src.rank, src.alpha, src.name, src.zo_sigma)
        return new

    def save(self, aid: int, name: str) -> str:
        self._get(aid).name = name
        path = self._path(name)
        from .policy import trusted
        with trusted():                      # the adapter store writes on the inferlet's behalf
            self.drivers[0].save_adapter(aid, path)
        return path

    def load(self, owner: str, name: str) -> int:
        self._supported()
        path = self._path(name)
        if not os.path.exists(path):
            raise AdapterError(f"no saved adapter {name!r}")
        from .policy import trusted
        with self._lock, trusted():
            aid = next(self._ids)
            for d in self.drivers:
                d.load_adapter(aid, path)
            a = self.drivers[0].adapters[aid]
            self.adapters[aid] = AdapterInfo(aid, owner, a.rank, a.alpha, name)
        return aid

    def release_owner(self, owner: str) -> None:
        for aid in [a.id for a in self.adapters.values() if a.owner == owner]:
            self.destroy(aid)

    # ---- zeroth-order optimisation
    def zo_init(self, aid: int, sigma: float) -> None:
        self._get(aid).zo_sigma = float(sigma)

    def zo_perturb(self, aid: int, seed: int, sign: float = 1.0) -> None:
        """params += sign * sigma * N(seed): evaluate a direction (call again with -sign to undo)."""
        info = self._get(aid)
        for d in self.drivers:
            d.zo_apply(aid, seed, sign * info.zo_sigma)

    def zo_update(self, aid: int, seeds: List[int], scores: List[float], lr: float) -> None:
        """Evolution-strategies step: params += lr / (n * sigma) * sum_i score_i * N(seed_i)."""
        info = self._get(aid)
        if len(seeds) != len(scores) or not seeds:
            raise AdapterError("seeds and scores must have the same non-zero length")
        if info.zo_sigma <= 0:
            raise AdapterError("call zo_init first")
        mean = sum(scores) / len(scores)
        for s, sc in zip(seeds, scores):
            coeff = lr * (sc - mean) / (len(seeds) * info.zo_sigma)
            if coeff:
                for d in self.drivers:
                    d.zo_apply(aid, s, coeff)
