"""Encoded media clips of one model.

An image or video enters a context as a run of placeholder tokens (`driver.schema.media_tokens`): one per row of
the vision encoder's output. The clip itself is encoded once by every driver replica of the model and stays on
the device under a small integer slot; forward requests name (slot, first row, count) for the placeholder rows
they carry, and the driver writes those encoder rows over the token embeddings. Slots are content-addressed -
the same pixels give the same slot, hence the same placeholders, hence shared KV pages through the ordinary
page hashes - and reference counted by the contexts (snapshots included) whose lineage holds the clip.

Counterpart of the media interface of the reference's host API and the image / audio CSR side channel of its
forward request (runtime/src/api/media.rs, runtime/src/inference/request.rs:657-988).
"""
from __future__ import annotations

import hashlib
import threading
from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Set, Tuple

import numpy as np

from ..driver.schema import MEDIA_ROWS, MEDIA_SLOTS, MEDIA_TOKEN_BASE, media_tokens


@dataclass
class MediaEntry:
    slot: int
    key: bytes
    kind: str
    rows: int
    refs: int = 0


class MediaRegistry:
    def __init__(self, drivers: Sequence):
        self.drivers = list(drivers)
        self.lock = threading.RLock()
        self.by_key: Dict[bytes, MediaEntry] = {}
        self.by_slot: Dict[int, MediaEntry] = {}
        self.of_context: Dict[int, Set[int]] = {}
        self._next = 0
        self._free: List[int] = []
        self.counters = {"encoded": 0, "shared": 0, "released": 0}

    @staticmethod
    def content_key(kind: str, patches: np.ndarray, grids) -> bytes:
        h = hashlib.blake2b(digest_size=16)
        h.update(kind.encode())
        h.update(np.asarray(grids, dtype=np.int32).tobytes())
        h.update(np.ascontiguousarray(patches, dtype=np.float32).tobytes())
        return h.digest()

    def put(self, ctx_id: int, kind: str, patches: np.ndarray, grids: Sequence[Tuple[int, int, int]]) -> List[int]:
        """Encode a clip (or find it encoded already), tie it to the context, return its placeholder tokens."""
        key = self.content_key(kind, patches, grids)
        with self.lock:
            e = self.by_key.get(key)
            if e is None:
                if self._free:
                    slot = self._free.pop()
                elif self._next < MEDIA_SLOTS:
                    slot, self._next = self._next, self._next + 1
                else:
                    raise RuntimeError("out of media slots")
                rows = {int(d.put_media(slot, kind, patches, grids)) for d in self.drivers}
                if len(rows) != 1 or not 0 < next(iter(rows)) <= MEDIA_ROWS:
                    for d in self.drivers:
                        d.release_media(slot)
                    self._free.append(slot)
                    raise RuntimeError(f"drivers disagree on the clip's size, or it is out of range: {sorted(rows)} rows")
                e = self.by_key[key] = self.by_slot[slot] = MediaEntry(slot, key, kind, rows.pop())
                self.counters["encoded"] += 1
            else:
                self.counters["shared"] += 1
            self._attach(ctx_id, e)
            return media_tokens(e.slot, e.rows)

    def _attach(self, ctx_id: int, e: MediaEntry) -> None:
        held = self.of_context.setdefault(ctx_id, set())
        if e.slot not in held:
            held.add(e.slot)
            e.refs += 1

    def fork(self, src_ctx: int, dst_ctx: int) -> None:
        with self.lock:
            for slot in list(self.of_context.get(src_ctx, ())):
                self._attach(dst_ctx, self.by_slot[slot])

    def drop(self, ctx_id: int) -> None:
        with self.lock:
            for slot in self.of_context.pop(ctx_id, ()):
                e = self.by_slot[slot]
                e.refs -= 1
                if e.refs <= 0:
                    del self.by_slot[slot], self.by_key[e.key]
                    self._free.append(slot)
                    self.counters["released"] += 1
                    for d in self.drivers:
                        try:
                            d.release_media(slot)
                        except Exception:  # noqa: BLE001 - a dead driver has nothing left to release
                            pass

    def stats(self) -> dict:
        with self.lock:
            return dict(self.counters, resident=len(self.by_slot), rows=sum(e.rows for e in self.by_slot.values()))


def is_media_token(tok: int) -> bool:
    return tok >= MEDIA_TOKEN_BASE
