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
from concurrent.futures import ThreadPoolExecutor
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
    ready: object = None      # runtime.inference.Future: set when every driver holds the encoded rows (or with the error)


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
        # encoders run off the caller's thread: an inferlet's coroutine appends the placeholders at once and only its
        # next forward pass waits for the rows (`MediaEntry.ready`)
        self._pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="pie-media")

    @staticmethod
    def content_key(kind: str, patches: np.ndarray, grids) -> bytes:
        h = hashlib.blake2b(digest_size=16)
        h.update(kind.encode())
        h.update(np.asarray(grids, dtype=np.int32).tobytes())
        h.update(np.ascontiguousarray(patches, dtype=np.float32).tobytes())
        return h.digest()

    def put(self, ctx_id: int, kind: str, patches: np.ndarray, grids: Sequence[Tuple[int, int, int]], rows: int):
        """Tie a clip of `rows` encoder rows to the context and return (its placeholder tokens, its entry). A clip
        that is not resident yet is handed to the drivers on the registry's worker thread; `entry.ready` completes
        when they hold it. Nothing here waits for an encoder."""
        from .inference import Future
        if not 0 < rows <= MEDIA_ROWS:
            raise ValueError(f"a clip of {rows} rows is outside the placeholder range")
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
                e = self.by_key[key] = self.by_slot[slot] = MediaEntry(slot, key, kind, rows, ready=Future())
                self.counters["encoded"] += 1
                self._pool.submit(self._encode, e, np.ascontiguousarray(patches, dtype=np.float32), [tuple(g) for g in grids])
            else:
                if e.rows != rows:
                    raise RuntimeError(f"clip is resident with {e.rows} rows, caller expects {rows}")
                self.counters["shared"] += 1
            self._attach(ctx_id, e)          # the reference is taken before the encoder runs: nobody frees the slot meanwhile
            return media_tokens(e.slot, e.rows), e

    def _encode(self, e: MediaEntry, patches: np.ndarray, grids) -> None:
        try:
            got = {int(d.put_media(e.slot, e.kind, patches, grids)) for d in self.drivers}
            if got != {e.rows}:
                raise RuntimeError(f"encoder gave {sorted(got)} rows for a clip planned with {e.rows}")
            e.ready.set(True)
        except BaseException as exc:  # noqa: BLE001 - the waiting forward pass gets the error
            with self.lock:         # the same content may be tried again; the contexts that hold this entry keep its slot until they go
                if self.by_key.get(e.key) is e:
                    del self.by_key[e.key]
            e.ready.set(None, exc)

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
                    del self.by_slot[slot]
                    if self.by_key.get(e.key) is e:
                        del self.by_key[e.key]
                    self._free.append(slot)
                    self.counters["released"] += 1
                    # after the encoder (same single worker): a clip dropped while it was being encoded is released too
                    self._pool.submit(self._release, slot)

    def _release(self, slot: int) -> None:
        with self.lock:
            if slot in self.by_slot:        # taken again meanwhile: that clip's rows now live there
                return
        for d in self.drivers:
            try:
                d.release_media(slot)
            except Exception:  # noqa: BLE001 - a dead driver has nothing left to release
                pass

    def drain(self, timeout: float = 30.0) -> None:
        """Wait until the worker has run everything queued so far (tests, shutdown)."""
        self._pool.submit(lambda: None).result(timeout)

    def close(self) -> None:
        self._pool.shutdown(wait=False, cancel_futures=True)

    def stats(self) -> dict:
        with self.lock:
            return dict(self.counters, resident=len(self.by_slot), rows=sum(e.rows for e in self.by_slot.values()))


def is_media_token(tok: int) -> bool:
    return tok >= MEDIA_TOKEN_BASE
