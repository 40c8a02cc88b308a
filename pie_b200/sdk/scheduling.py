"""WIT `scheduling` interface: read-only view of the KV market for the calling inferlet.
price() is the constant 1.0 in the reference (runtime/src/api/scheduling.rs:12-59)."""
from __future__ import annotations

from . import host


def price() -> float:
    return 1.0


def rent(ctx) -> float:
    m = getattr(ctx._entry, "market", None)
    return m.rent_of(ctx.id) if m is not None else ctx._entry.ctxm.effective_pages(ctx.id)


def dividend(model) -> float:
    m = getattr(model._entry, "market", None)
    return m.last_dividend(host.proc().id) if m is not None else 0.0


def latency(ctx) -> float:
    s = ctx._entry.schedulers[0].stats
    return s["last_latency_us"] / 1e6


def balance(model) -> float:
    m = getattr(model._entry, "market", None)
    return m.balance(host.proc().id) if m is not None else 0.0
