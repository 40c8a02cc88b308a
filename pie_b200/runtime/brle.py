"""Binary run-length encoding of boolean vectors.

A BRLE vector is a list of run lengths; runs alternate False, True, False, ... starting with a
(possibly empty) run of False. Attention masks (one vector per query token over the KV
positions) and logit masks (one vector over the vocabulary) travel in this form.
Same encoding as the reference (driver/bridge/src/brle.rs:1-36); the native implementation
used on the hot path lives in csrc/host/brle.hpp, this module is the portable fallback and
the oracle of its tests.
"""
from __future__ import annotations

from typing import Iterable, List, Sequence

import numpy as np


def encode(bits: Sequence[bool]) -> List[int]:
    a = np.asarray(bits, dtype=bool)
    if a.size == 0:
        return []
    change = np.flatnonzero(a[1:] != a[:-1]) + 1
    bounds = np.concatenate([[0], change, [a.size]])
    runs = np.diff(bounds).tolist()
    if a[0]:
        runs.insert(0, 0)
    return runs


def decode(runs: Iterable[int], size: int = -1, tail: bool = False) -> np.ndarray:
    runs = list(runs)
    total = sum(runs)
    n = total if size < 0 else size
    out = np.full(n, tail, dtype=bool)
    pos = 0
    for i, r in enumerate(runs):
        if pos >= n:
            break
        end = min(n, pos + r)
        out[pos:end] = bool(i & 1)
        pos = end
    return out


def all_true(n: int) -> List[int]:
    return [0, n]


def all_false(n: int) -> List[int]:
    return [n]


def length(runs: Iterable[int]) -> int:
    return sum(runs)


def count_true(runs: Sequence[int]) -> int:
    return sum(runs[1::2])


def range_mask(n: int, start: int, end: int) -> List[int]:
    """True on [start, end) of n positions."""
    start, end = max(0, start), min(n, end)
    if end <= start:
        return [n]
    out = [start, end - start]
    if end < n:
        out.append(n - end)
    return out


def normalise(runs: Sequence[int]) -> List[int]:
    """Merge zero-length interior runs so that equal vectors have equal encodings."""
    out: List[int] = []
    for i, r in enumerate(runs):
        if i == 0:
            out.append(r)
        elif r == 0 and i != len(runs) - 1 and out:
            # a zero-length run joins its neighbours: pop the previous run and extend it later
            out.append(0)
        else:
            out.append(r)
    # collapse patterns [a, 0, b] -> [a + b]
    res: List[int] = []
    for r in out:
        if len(res) >= 2 and res[-1] == 0 and len(res) > 1:
            res.pop()
            res[-1] += r
        else:
            res.append(r)
    while len(res) > 1 and res[-1] == 0:
        res.pop()
    return res


def logical_and(a: Sequence[int], b: Sequence[int]) -> List[int]:
    n = max(length(a), length(b))
    return encode(decode(a, n) & decode(b, n))


def append(runs: List[int], value: bool, count: int = 1) -> List[int]:
    runs = list(runs)
    if count <= 0:
        return runs
    if not runs:
        return [count] if not value else [0, count]
    last_is_true = (len(runs) - 1) & 1 == 1
    if last_is_true == bool(value):
        runs[-1] += count
    else:
        runs.append(count)
    return runs


def is_causal_prefix(runs: Sequence[int], visible: int) -> bool:
    """True when the vector is exactly `visible` ones (a causal row) possibly followed by zeros."""
    r = [x for x in runs]
    if len(r) >= 2 and r[0] == 0 and r[1] == visible and all(x == 0 for x in r[3::2]):
        return True
    return False


def droppable_pages(rows: Sequence[Sequence[int]], page_size: int, num_pages: int) -> np.ndarray:
    """Pages whose positions are masked out in every row (candidates for page trim)."""
    vis = np.zeros(num_pages * page_size, dtype=bool)
    for r in rows:
        d = decode(r, num_pages * page_size)
        vis |= d
    return ~vis.reshape(num_pages, page_size).any(axis=1)


def remove_pages(runs: Sequence[int], drop: np.ndarray, page_size: int) -> List[int]:
    """The vector without the positions of the pages flagged in `drop` (page trim re-indexing)."""
    n = max(length(runs), len(drop) * page_size)
    bits = decode(runs, n)
    keep = np.ones(n, dtype=bool)
    keep[:len(drop) * page_size] = ~np.repeat(np.asarray(drop, dtype=bool), page_size)
    return encode(bits[keep])


try:  # native implementations (csrc/host/brle.hpp) replace the hot entry points when built
    from .._C import pie_host as _native

    def encode(bits) -> List[int]:  # noqa: F811
        return _native.brle_encode(np.ascontiguousarray(bits, dtype=bool))

    def decode(runs, size: int = -1, tail: bool = False) -> np.ndarray:  # noqa: F811
        return _native.brle_decode(list(runs), size, tail)

    def logical_and(a, b) -> List[int]:  # noqa: F811
        return _native.brle_and(list(a), list(b))

    def droppable_pages(rows, page_size: int, num_pages: int) -> np.ndarray:  # noqa: F811
        return _native.brle_droppable_pages([list(r) for r in rows], page_size, num_pages)

    NATIVE = True
except ImportError:  # pragma: no cover
    NATIVE = False
