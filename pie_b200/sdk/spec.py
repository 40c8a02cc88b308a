"""Custom speculators: an inferlet-side drafter whose tokens ride along as speculative inputs
and are verified in the same forward pass (sdk/python/src/inferlet/spec.py:19-57)."""
from __future__ import annotations

from typing import List, Protocol, Tuple


class Speculator(Protocol):
    def draft(self) -> Tuple[List[int], List[int]]:
        """Return (draft tokens, positions); positions may be empty for 'consecutive'."""

    def accept(self, tokens: List[int]) -> None: ...

    def rollback(self, n: int) -> None: ...

    def reset(self) -> None: ...


class NGramSpeculator:
    """Drafts the continuation that followed the most recent occurrence of the last n tokens."""

    def __init__(self, history: List[int], n: int = 2, max_draft: int = 4):
        self.hist, self.n, self.max_draft = list(history), n, max_draft

    def draft(self):
        h = self.hist
        if len(h) <= self.n:
            return [], []
        key = h[-self.n:]
        for i in range(len(h) - self.n - 1, -1, -1):
            if h[i:i + self.n] == key:
                return h[i + self.n:i + self.n + self.max_draft], []
        return [], []

    def accept(self, tokens):
        self.hist.extend(tokens)

    def rollback(self, n):
        del self.hist[len(self.hist) - n:]

    def reset(self):
        self.hist.clear()
