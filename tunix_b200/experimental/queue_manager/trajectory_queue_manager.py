"""Grouped trajectory queue with in-flight acknowledgement and a staleness filter
(tunix/experimental/queue_manager/trajectory_queue_manager.py).

Producers `put(group_id, item, policy_version)`; a group is released to consumers once `group_size` items have
arrived. A consumer `get()`s a group, which then counts as in flight until it is `ack`ed; `nack` (or a consumer
that disappears: `requeue_expired`) puts it back at the front. Groups whose oldest item is more than
`max_staleness` policy versions behind the current one are dropped on the way out. With `ordered=True` groups
are released in the order their first item arrived (batch-ordered variant), otherwise in completion order."""
from __future__ import annotations

import collections
import threading
import time
from typing import Any, Optional


class TrajectoryQueueManager:
    def __init__(self, group_size: int, max_staleness: Optional[int] = None, ordered: bool = False, inflight_timeout_s: float = 600.0):
        self.group_size, self.max_staleness, self.ordered = group_size, max_staleness, ordered
        self.inflight_timeout_s = inflight_timeout_s
        self._open: "collections.OrderedDict[str, list]" = collections.OrderedDict()
        self._ready: collections.deque = collections.deque()
        self._inflight: dict = {}
        self._cv = threading.Condition()
        self.current_version = 0
        self.dropped_stale = 0
        self._closed = False

    def set_policy_version(self, v: int) -> None:
        with self._cv:
            self.current_version = v

    def put(self, group_id: str, item: Any, policy_version: int = 0) -> None:
        with self._cv:
            if self._closed:
                raise RuntimeError("queue is closed")
            bucket = self._open.setdefault(group_id, [])
            bucket.append((item, policy_version))
            if self.ordered:
                while self._open:
                    gid, b = next(iter(self._open.items()))
                    if len(b) < self.group_size:
                        break
                    self._open.pop(gid)
                    self._ready.append((gid, b))
            elif len(bucket) >= self.group_size:
                self._ready.append((group_id, self._open.pop(group_id)))
            self._cv.notify_all()

    def _stale(self, bucket) -> bool:
        return self.max_staleness is not None and self.current_version - min(v for _, v in bucket) > self.max_staleness

    def get(self, timeout: Optional[float] = None) -> Optional[tuple]:
        """(group_id, [items]) of the next fresh group, or None on timeout / closed-and-empty."""
        deadline = None if timeout is None else time.monotonic() + timeout
        with self._cv:
            while True:
                while self._ready:
                    gid, bucket = self._ready.popleft()
                    if self._stale(bucket):
                        self.dropped_stale += 1
                        continue
                    self._inflight[gid] = (bucket, time.monotonic())
                    return gid, [it for it, _ in bucket]
                if self._closed:
                    return None
                left = None if deadline is None else deadline - time.monotonic()
                if left is not None and left <= 0:
                    return None
                self._cv.wait(left)

    def ack(self, group_id: str) -> None:
        with self._cv:
            self._inflight.pop(group_id)

    def nack(self, group_id: str) -> None:
        with self._cv:
            bucket, _ = self._inflight.pop(group_id)
            self._ready.appendleft((group_id, bucket))
            self._cv.notify_all()

    def requeue_expired(self) -> int:
        now, n = time.monotonic(), 0
        with self._cv:
            for gid in [g for g, (_, t) in self._inflight.items() if now - t > self.inflight_timeout_s]:
                bucket, _ = self._inflight.pop(gid)
                self._ready.appendleft((gid, bucket))
                n += 1
            if n:
                self._cv.notify_all()
        return n

    def close(self) -> None:
        with self._cv:
            self._closed = True
            self._cv.notify_all()

    @property
    def num_inflight(self) -> int:
        return len(self._inflight)

    @property
    def num_ready(self) -> int:
        return len(self._ready)
