"""In-process data queues between the rollout producer and the trainer (tunix/rl/queue/data_queue.py:27-68)."""
from __future__ import annotations

import abc
import queue
from typing import Generic, Optional, TypeVar

T = TypeVar("T")


class AbstractDataQueue(abc.ABC, Generic[T]):
    @abc.abstractmethod
    def put(self, item: T) -> None: ...
    @abc.abstractmethod
    def get(self, block: bool = True, timeout: Optional[float] = None) -> T: ...
    @abc.abstractmethod
    def qsize(self) -> int: ...
    @abc.abstractmethod
    def close(self) -> None: ...


class SimpleDataQueue(AbstractDataQueue[T]):
    def __init__(self, maxsize: int = 0):
        self._q: queue.Queue = queue.Queue(maxsize=maxsize)

    def put(self, item: T) -> None:
        self._q.put(item)

    def get(self, block: bool = True, timeout: Optional[float] = None) -> T:
        return self._q.get(block=block, timeout=timeout)

    def qsize(self) -> int:
        return self._q.qsize()

    def close(self) -> None:
        while not self._q.empty():
            try:
                self._q.get_nowait()
            except queue.Empty:
                break
