"""Async grouping of trajectory items by prompt until G arrive (tunix/rl/agentic/queue_manager/group_queue_manager.py)."""
from __future__ import annotations

import asyncio
import collections
from typing import Any, Hashable, Optional


class GroupQueueManager:
    def __init__(self, *, group_size: int, max_open_buckets: Optional[int] = None):
        self.group_size = group_size
        self.max_open_buckets = max_open_buckets
        self._buckets: dict = collections.OrderedDict()
        self._ready: collections.deque = collections.deque()
        self._cond = asyncio.Condition()
        self._exc: Optional[BaseException] = None
        self._closed = False

    async def put(self, item: Any, group_key: Optional[Hashable] = None) -> None:
        key = group_key if group_key is not None else getattr(item, "group_id", None)
        async with self._cond:
            while (self.max_open_buckets and key not in self._buckets and len(self._buckets) >= self.max_open_buckets
                   and not self._closed):
                await self._cond.wait()
            b = self._buckets.setdefault(key, [])
            b.append(item)
            if len(b) >= self.group_size:
                self._ready.append(self._buckets.pop(key))
            self._cond.notify_all()

    async def put_exception(self, exc: BaseException) -> None:
        async with self._cond:
            self._exc = exc
            self._cond.notify_all()

    async def close(self) -> None:
        async with self._cond:
            self._closed = True
            self._cond.notify_all()

    async def get_batch(self, n_groups: int = 1) -> Optional[list]:
        """Wait for `n_groups` complete groups; returns fewer (or None) only after close()."""
        async with self._cond:
            while len(self._ready) < n_groups and self._exc is None and not self._closed:
                await self._cond.wait()
            if self._exc is not None:
                e, self._exc = self._exc, None
                raise e
            if not self._ready:
                return None
            out = [self._ready.popleft() for _ in range(min(n_groups, len(self._ready)))]
            self._cond.notify_all()
            return out

    @property
    def open_buckets(self) -> int:
        return len(self._buckets)
