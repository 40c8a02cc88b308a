"""KV market: admission of processes and pricing of contended KV pages.

Every process holds two wallets per model: a token budget (debited as its contexts grow) and a
credit balance. Credits are endowed at admission in proportion to the pages the process may
claim. After every batch the market ticks: when the page pool is contended the clearing price is
the lowest bid among the contexts in the batch, each context in the batch pays rent
(price x effective pages, shared pages split between holders), and the collected rent is paid
out as dividends in proportion to endowments. A process whose balance went negative has
defaulted: its contexts are the first eviction victims (then lowest bid, then newest).
Admission gate: the sum of claims must stay below capacity x oversubscription factor + slack.

Behavioural counterpart of runtime/src/context/sched.rs:85-118 (wallets), :182-279 (admission),
:432-612 (tick), :881-938 (victim order); `scheduling` WIT queries read these numbers.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional


@dataclass
class Wallet:
    endowment_pages: float
    credits: float
    tokens_left: Optional[int] = None
    rent_paid: float = 0.0
    dividends: float = 0.0
    last_dividend: float = 0.0


class Market:
    def __init__(self, capacity_pages: int, default_endowment_pages: int = 64, oversubscription: float = 4.0,
                 slack_pages: int = 0, contention_threshold: float = 0.9):
        self.capacity = capacity_pages
        self.default_endowment = default_endowment_pages
        self.oversubscription = oversubscription
        self.slack = slack_pages
        self.contention_threshold = contention_threshold
        self.wallets: Dict[str, Wallet] = {}
        self.claims: Dict[str, float] = {}
        self.waiting: List[tuple] = []           # (owner, claim, callback)
        self.lock = threading.Lock()
        self.clearing_price = 0.0
        self.last_rent: Dict[int, float] = {}    # context id -> rent of the last tick
        self.ticks = 0
        self.total_rent = 0.0
        self.total_dividends = 0.0

    # ------------------------------------------------------------------ admission
    def _limit(self) -> float:
        return self.capacity * self.oversubscription + self.slack

    def try_admit(self, owner: str, claim_pages: Optional[float] = None, token_budget: Optional[int] = None,
                  on_admit: Optional[Callable[[], None]] = None) -> bool:
        """Admit `owner` if its claim fits; otherwise queue it (drained in order on release)."""
        claim = float(self.default_endowment if claim_pages is None else claim_pages)
        with self.lock:
            if owner in self.wallets:
                return True
            if not self.waiting and sum(self.claims.values()) + claim <= self._limit():
                self._admit(owner, claim, token_budget)
                return True
            self.waiting.append((owner, claim, token_budget, on_admit))
            return False

    def _admit(self, owner, claim, token_budget) -> None:
        self.claims[owner] = claim
        self.wallets[owner] = Wallet(endowment_pages=claim, credits=claim, tokens_left=token_budget)

    def release(self, owner: str) -> None:
        """The process ended: free its claim and admit queued processes that now fit (in order:
        a large claim at the head is a drain barrier for the ones behind it)."""
        cbs = []
        with self.lock:
            self.claims.pop(owner, None)
            self.wallets.pop(owner, None)
            while self.waiting:
                o, claim, budget, cb = self.waiting[0]
                if sum(self.claims.values()) + claim > self._limit():
                    break
                self.waiting.pop(0)
                self._admit(o, claim, budget)
                if cb:
                    cbs.append(cb)
        for cb in cbs:
            cb()

    # ------------------------------------------------------------------ accounting
    def debit_tokens(self, owner: str, n: int) -> bool:
        """Token wallet: returns False when the budget is exhausted (pins are then refused)."""
        with self.lock:
            w = self.wallets.get(owner)
            if w is None or w.tokens_left is None:
                return True
            w.tokens_left -= n
            return w.tokens_left >= 0

    def budget_exhausted(self, owner: str) -> bool:
        with self.lock:
            w = self.wallets.get(owner)
            return w is not None and w.tokens_left is not None and w.tokens_left <= 0

    def tick(self, used_pages: int, batch: Iterable[tuple]) -> float:
        """One market step after a batch. `batch` = (context id, owner, bid, effective pages) of the
        contexts that were in the batch. Returns the clearing price."""
        batch = list(batch)
        with self.lock:
            self.ticks += 1
            contended = used_pages >= self.contention_threshold * self.capacity
            price = min((b for _, _, b, _ in batch), default=0.0) if contended and batch else 0.0
            self.clearing_price = price
            self.last_rent = {}
            collected = 0.0
            for cid, owner, _bid, pages in batch:
                rent = price * pages
                self.last_rent[cid] = rent
                w = self.wallets.get(owner)
                if w is not None and rent:
                    w.credits -= rent
                    w.rent_paid += rent
                    collected += rent
            self.total_rent += collected
            total_endow = sum(w.endowment_pages for w in self.wallets.values())
            for w in self.wallets.values():
                w.last_dividend = collected * w.endowment_pages / total_endow if total_endow else 0.0
                w.credits += w.last_dividend
                w.dividends += w.last_dividend
            self.total_dividends += collected if total_endow else 0.0
            return price

    # ------------------------------------------------------------------ queries
    def balance(self, owner: str) -> float:
        with self.lock:
            w = self.wallets.get(owner)
            return w.credits if w else 0.0

    def last_dividend(self, owner: str) -> float:
        with self.lock:
            w = self.wallets.get(owner)
            return w.last_dividend if w else 0.0

    def rent_of(self, cid: int) -> float:
        with self.lock:
            return self.last_rent.get(cid, 0.0)

    def defaulted(self, owner: str) -> bool:
        with self.lock:
            w = self.wallets.get(owner)
            return w is not None and w.credits < 0

    def victim_key(self, owner: str, bid: float, created_seq: int) -> tuple:
        """Sort key: smallest = evicted first (defaulted, then lowest bid, then newest)."""
        return (0 if self.defaulted(owner) else 1, bid, -created_seq)

    def conservation_error(self) -> float:
        """Credits are conserved: sum(credits) = sum(endowments) for the admitted processes."""
        with self.lock:
            return abs(sum(w.credits for w in self.wallets.values()) -
                       sum(w.endowment_pages for w in self.wallets.values()))
