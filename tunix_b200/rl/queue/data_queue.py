"""The hand-over point between the thread that produces rollout batches and the training loop that consumes them
(the role of tunix/rl/queue/data_queue.py:27-68).

`SimpleDataQueue` is a bounded FIFO on a deque and one condition variable rather than a wrapper around
`queue.Queue`, for the one thing the standard queue cannot do: `close()` wakes every thread blocked in `put` or
`get`, so a learner that stops early (an exception in the training loop, `max_steps` reached) never leaves its
producer thread parked on a full queue. After `close()` a `put` is dropped and a `get` on the drained queue
raises `queue.Empty`."""
from __future__ import annotations

import abc
import collections
import queue
import threading
import time
from typing import Generic, Optional, TypeVar

T = TypeVar("T")


class AbstractDataQueue(abc.ABC, Generic[T]):
    """What the learner needs of a queue; a multi-process or multi-host queue implements the same four calls."""

    @abc.abstractmethod
    def put(self, item: T) -> None:
        """Append `item`, waiting for room when the queue is bounded and full."""

    @abc.abstractmethod
    def get(self, block: bool = True, timeout: Optional[float] = None) -> T:
        """Remove and return the oldest item; `queue.Empty` when there is none (in time)."""

    @abc.abstractmethod
    def qsize(self) -> int:
        """Items waiting right now."""

    @abc.abstractmethod
    def close(self) -> None:
        """Drop what is waiting and release every blocked caller."""


class SimpleDataQueue(AbstractDataQueue[T]):
    def __init__(self, maxsize: int = 0):
        self._items: collections.deque = collections.deque()
        self._cap = int(maxsize) if maxsize and maxsize > 0 else 0
        self._cv = threading.Condition()
        self._closed = False

    @property
    def closed(self) -> bool:
        return self._closed

    def put(self, item: T) -> None:
        with self._cv:
            while self._cap and len(self._items) >= self._cap and not self._closed:
                self._cv.wait()
            if self._closed:
                return
            self._items.append(item)
            self._cv.notify_all()

    def get(self, block: bool = True, timeout: Optional[float] = None) -> T:
        deadline = None if timeout is None else time.monotonic() + timeout
        with self._cv:
            while not self._items:
                if not block or self._closed:
                    raise queue.Empty
                left = None if deadline is None else deadline - time.monotonic()
                if left is not None and left <= 0:
                    raise queue.Empty
                self._cv.wait(left)
            item = self._items.popleft()
            self._cv.notify_all()
            return item

    def qsize(self) -> int:
        with self._cv:
            return len(self._items)

    def close(self) -> None:
        with self._cv:
            self._closed = True
            self._items.clear()
            self._cv.notify_all()
