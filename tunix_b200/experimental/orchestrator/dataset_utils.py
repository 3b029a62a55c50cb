"""Prompt datasets for the orchestrator (tunix/experimental/orchestrator/dataset_utils.py:35-167): how many prompt
groups a run will ask for, and reading the dataset on a background thread so that tokenisation or file reads never
stall the dispatch loop.

`PrefetchIterator` yields `(index, item)` with the indices of `enumerate(dataset)`, skips a resumed run's prefix
without handing it out, keeps at most `prefetch_size` items ahead, forwards the dataset's exception to the consumer
at the position where it happened, and closes the underlying generator when the consumer stops early.
`iter_dataset_async` is the same thing for an asyncio consumer."""
from __future__ import annotations

import asyncio
import queue
import threading
from typing import AsyncIterator, Iterable, Iterator, TypeVar

T = TypeVar("T")
_END = object()


def total_prompt_groups(max_steps: int, batch_size: int, max_staleness: int = 0) -> int:
    """Prompt groups to provide for `max_steps` updates: off-policy runs dispatch ahead of the trainer, so they are
    given a look-ahead margin (at least 6 steps, 4 per step of allowed staleness, a quarter of the run)."""
    extra = max(max_staleness * 4, 6, max_steps // 4) if max_staleness > 0 else 0
    return (max_steps + extra) * batch_size


class PrefetchIterator(Iterator):
    def __init__(self, dataset: Iterable[T], *, skip_count: int = 0, prefetch_size: int = 1):
        self._fast = None
        if isinstance(dataset, (list, tuple)):              # nothing to overlap: index directly
            self._fast = iter(range(max(0, skip_count), len(dataset)))
            self._data = dataset
            return
        self._q: "queue.Queue" = queue.Queue(maxsize=max(1, prefetch_size))
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._produce, args=(dataset, max(0, skip_count)), name="prompt-prefetch", daemon=True)
        self._thread.start()

    def _put(self, item) -> bool:
        while not self._stop.is_set():
            try:
                self._q.put(item, timeout=0.05)
                return True
            except queue.Full:
                continue
        return False

    def _produce(self, dataset, skip: int) -> None:
        it = iter(dataset)
        try:
            for idx, item in enumerate(it):
                if self._stop.is_set():
                    return
                if idx < skip:
                    continue
                if not self._put((idx, item)):
                    return
            self._put(_END)
        except BaseException as e:
            self._put(e)
        finally:
            close = getattr(it, "close", None)
            if callable(close):
                close()

    def __iter__(self):
        return self

    def __next__(self):
        if self._fast is not None:
            i = next(self._fast)
            return i, self._data[i]
        if self._stop.is_set():
            raise StopIteration
        item = self._q.get()
        if item is _END:
            self._stop.set()
            raise StopIteration
        if isinstance(item, BaseException):
            self._stop.set()
            raise item
        return item

    def close(self) -> None:
        if self._fast is None:
            self._stop.set()
            self._thread.join(5.0)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


async def iter_dataset_async(dataset: Iterable[T], *, skip_count: int = 0, prefetch_size: int = 1) -> AsyncIterator:
    it = PrefetchIterator(dataset, skip_count=skip_count, prefetch_size=prefetch_size)
    loop = asyncio.get_running_loop()
    try:
        while True:
            item = next(it, _END) if it._fast is not None else await loop.run_in_executor(None, next, it, _END)
            if item is _END:
                return
            yield item
    finally:
        it.close()
