"""Inter-inferlet messaging: point-to-point queues (push / pull) and topics (broadcast /
subscribe). Counterpart of runtime/src/messaging.rs:1-90 and the `messaging` WIT interface."""
from __future__ import annotations

import asyncio
from collections import defaultdict, deque
from typing import Deque, Dict, List


class Subscription:
    def __init__(self, hub: "Messaging", topic: str):
        self.hub, self.topic = hub, topic
        self.queue: "asyncio.Queue[str]" = asyncio.Queue()
        self.active = True

    async def get(self) -> str:
        return await self.queue.get()

    def get_nowait(self):
        try:
            return self.queue.get_nowait()
        except asyncio.QueueEmpty:
            return None

    def unsubscribe(self) -> None:
        if self.active:
            self.active = False
            self.hub._subs[self.topic].remove(self)


class Messaging:
    """Lives on the runtime's event loop; all methods are called from inferlet coroutines."""

    def __init__(self):
        self._queues: Dict[str, Deque[str]] = defaultdict(deque)
        self._waiters: Dict[str, Deque[asyncio.Future]] = defaultdict(deque)
        self._subs: Dict[str, List[Subscription]] = defaultdict(list)

    def push(self, topic: str, message: str) -> None:
        waiters = self._waiters[topic]
        while waiters:
            w = waiters.popleft()
            if not w.done():
                w.set_result(message)
                return
        self._queues[topic].append(message)

    async def pull(self, topic: str) -> str:
        q = self._queues[topic]
        if q:
            return q.popleft()
        fut = asyncio.get_running_loop().create_future()
        self._waiters[topic].append(fut)
        return await fut

    def broadcast(self, topic: str, message: str) -> None:
        for s in list(self._subs[topic]):
            s.queue.put_nowait(message)

    def subscribe(self, topic: str) -> Subscription:
        s = Subscription(self, topic)
        self._subs[topic].append(s)
        return s
