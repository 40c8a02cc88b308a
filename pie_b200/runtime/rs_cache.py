"""Recurrent-state slot pool for linear-attention / state-space layers: one slot per resident
context. A context's state is Unsupported (model has no recurrent layers), Empty (nothing
computed yet), Resident (slot holds the state that matches its KV length) or Missing (evicted or
invalidated: must be rebuilt by replaying the lineage).
Counterpart of runtime/src/context/rs_cache.rs:13-78.
"""
from __future__ import annotations

from enum import Enum
from typing import Dict, List, Optional

RS_FLAG_RESET = 1          # the driver must zero the slot before this pass


class RsState(Enum):
    UNSUPPORTED = 0
    EMPTY = 1
    RESIDENT = 2
    MISSING = 3


class RsCache:
    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self.free: List[int] = list(range(num_slots - 1, -1, -1))
        self.slot_of: Dict[int, int] = {}
        self.state: Dict[int, RsState] = {}

    @property
    def supported(self) -> bool:
        return self.num_slots > 0

    def state_of(self, ctx: int) -> RsState:
        if not self.supported:
            return RsState.UNSUPPORTED
        return self.state.get(ctx, RsState.EMPTY)

    def acquire(self, ctx: int) -> Optional[int]:
        """Slot of `ctx`, allocating one if needed; None when the pool is exhausted."""
        if not self.supported:
            return None
        if ctx in self.slot_of:
            return self.slot_of[ctx]
        if not self.free:
            return None
        s = self.free.pop()
        self.slot_of[ctx] = s
        self.state.setdefault(ctx, RsState.EMPTY)
        return s

    def flags_for_pass(self, ctx: int) -> int:
        """Flags the driver needs for the next pass of `ctx`; marks the state resident."""
        st = self.state_of(ctx)
        self.state[ctx] = RsState.RESIDENT
        return RS_FLAG_RESET if st in (RsState.EMPTY, RsState.MISSING) else 0

    def invalidate(self, ctx: int) -> None:
        """The state no longer matches the context (truncate, failed pass): rebuild by replay."""
        if ctx in self.state and self.supported:
            self.state[ctx] = RsState.MISSING

    def release(self, ctx: int) -> None:
        s = self.slot_of.pop(ctx, None)
        if s is not None:
            self.free.append(s)
        if self.state.get(ctx) == RsState.RESIDENT:
            self.state[ctx] = RsState.MISSING

    def forget(self, ctx: int) -> None:
        self.release(ctx)
        self.state.pop(ctx, None)

    def fork(self, src: int, dst: int) -> Optional[tuple]:
        """Give `dst` a slot holding a copy of `src`'s state: returns (src_slot, dst_slot) for the
        driver's slot copy, or None when there is nothing to copy."""
        if self.state_of(src) != RsState.RESIDENT:
            return None
        d = self.acquire(dst)
        if d is None:
            self.state[dst] = RsState.MISSING
            return None
        self.state[dst] = RsState.RESIDENT
        return self.slot_of[src], d
