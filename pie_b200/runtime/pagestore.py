"""Physical KV page pool and the content-addressed store of committed pages.

Committed pages are immutable and shared: a page is identified by the hash of its content
(tokens, positions, attention-mask rows, adapter seed) chained with the hash of the page before
it, so two contexts whose token prefixes agree resolve to the same chain of physical pages
(prefix caching and fork both fall out of this). Each node counts the contexts whose chain
passes through it; a page returns to the pool when the count reaches zero.

Behavioural counterpart of the reference's page store
(runtime/src/context/pagestore.rs:41-138 pool with double-free detection, :152-602 radix trie
with path-inclusive reference counts, :952-1006 chained content hash). Chained hashes make a
flat hash map equivalent to the trie: a node's key already encodes its whole path.
"""
from __future__ import annotations

import hashlib
import struct
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple


class PagePoolError(RuntimeError):
    pass


class PagePool:
    """Free list over `num_pages` physical page ids with double-free detection."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))
        self._is_free = [True] * num_pages
        self.double_free_count = 0

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self, n: int) -> Optional[List[int]]:
        if n > len(self._free):
            return None
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._is_free[p] = False
        return out

    def free(self, pages: Iterable[int]) -> None:
        for p in pages:
            if p < 0 or p >= self.num_pages:
                raise PagePoolError(f"page id {p} out of range")
            if self._is_free[p]:
                self.double_free_count += 1
                continue
            self._is_free[p] = True
            self._free.append(p)


def page_hash(prev: int, tokens: Sequence[int], positions: Sequence[int], mask_key: bytes = b"",
              adapter_seed: int = 0) -> int:
    """64-bit content hash of one full page chained to the previous page's hash."""
    h = hashlib.blake2b(digest_size=8)
    h.update(struct.pack("<QQI", prev & 0xFFFFFFFFFFFFFFFF, adapter_seed & 0xFFFFFFFFFFFFFFFF, len(tokens)))
    h.update(struct.pack(f"<{len(tokens)}I", *tokens))
    h.update(struct.pack(f"<{len(positions)}I", *positions))
    h.update(mask_key)
    return int.from_bytes(h.digest(), "little") or 1


@dataclass
class _Node:
    page: int
    parent: int          # chain hash of the previous page (0 = root)
    refcount: int = 0
    children: int = 0


class PyPageStore:
    """Per-driver store: pool + committed-page index (portable implementation)."""

    def __init__(self, num_pages: int):
        self.pool = PagePool(num_pages)
        self.nodes: Dict[int, _Node] = {}

    # ---- committed chains
    def lookup(self, chain_hash: int) -> Optional[int]:
        n = self.nodes.get(chain_hash)
        return None if n is None else n.page

    def extend(self, parent_hash: int, chain_hash: int, page: int) -> Tuple[int, bool]:
        """Attach a freshly filled working page as the committed node `chain_hash`.

        Returns (physical page to use, deduplicated). When a node with the same hash exists the
        caller's page is redundant: the existing page is shared and the caller frees its own.
        """
        node = self.nodes.get(chain_hash)
        if node is not None:
            node.refcount += 1
            return node.page, True
        self.nodes[chain_hash] = _Node(page=page, parent=parent_hash, refcount=1)
        if parent_hash in self.nodes:
            self.nodes[parent_hash].children += 1
        return page, False

    def acquire(self, chain: Sequence[int]) -> None:
        """A new holder (fork, snapshot, open) of every node on `chain`."""
        for h in chain:
            self.nodes[h].refcount += 1

    def release(self, chain: Sequence[int]) -> List[int]:
        """Drop one holder of every node of `chain`; returns the physical pages freed."""
        freed = []
        for h in reversed(chain):
            node = self.nodes.get(h)
            if node is None:
                continue
            node.refcount -= 1
            if node.refcount <= 0 and node.children == 0:
                freed.append(node.page)
                del self.nodes[h]
                parent = self.nodes.get(node.parent)
                if parent is not None:
                    parent.children -= 1
        self.pool.free(freed)
        return freed

    def would_free(self, chain: Sequence[int]) -> int:
        """Pages that releasing `chain` would return to the pool (tail nodes held only by it)."""
        n = 0
        for h in reversed(chain):
            node = self.nodes.get(h)
            if node is None or node.refcount > 1 or (node.children > (1 if n else 0)):
                break
            n += 1
        return n

    def prefix_len(self, hashes: Sequence[int]) -> int:
        """Number of leading chain hashes already present (prefix-cache hit length)."""
        n = 0
        for h in hashes:
            if h not in self.nodes:
                break
            n += 1
        return n

    def physical_ids(self, chain: Sequence[int]) -> List[int]:
        return [self.nodes[h].page for h in chain]

    def node_pages(self) -> List[int]:
        return [n.page for n in self.nodes.values()]

    def effective_pages(self, chain: Sequence[int], working: int) -> float:
        """Cost share of a context: shared pages are split between their holders."""
        return working + sum(1.0 / max(1, self.nodes[h].refcount) for h in chain if h in self.nodes)


py_page_hash = page_hash
try:  # the native store (csrc/host/pagestore.hpp) is the one used when the host module is built
    from .._C import pie_host as _native
    PageStore = _native.PageStore
    NATIVE = True

    def page_hash(prev: int, tokens, positions, mask_key: bytes = b"", adapter_seed: int = 0) -> int:  # noqa: F811
        return _native.page_hash(prev, list(tokens), list(positions), mask_key, adapter_seed)
except ImportError:  # pragma: no cover - exercised only without a compiler
    PageStore = PyPageStore
    NATIVE = False
