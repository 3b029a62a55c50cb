"""A writer thread behind a bounded queue (tunix/experimental/trajectory/async_writer.py:33-397).

Producers (rollout workers) hand over write tasks and go on; the thread applies them in order. When the queue is
full a producer waits (back-pressure instead of unbounded memory); a task that fails is logged and counted, the
writer goes on with the next one; `flush()` returns when everything queued so far has been applied; `close()` flushes,
stops the thread and is idempotent. Writers still open at interpreter exit are closed then, so that a crash-free
shutdown loses nothing."""
from __future__ import annotations

import abc
import atexit
import logging
import queue
import threading
import weakref
from typing import Generic, Optional, TypeVar

log = logging.getLogger(__name__)
_T = TypeVar("_T")
_STOP = object()
_live: "weakref.WeakSet" = weakref.WeakSet()


def _close_live_writers() -> None:
    for w in list(_live):
        try:
            w.close()
        except Exception:       # interpreter is going down: nothing useful left to do with the error
            pass


atexit.register(_close_live_writers)


class WriterClosedError(RuntimeError):
    pass


class AsyncWriter(abc.ABC, Generic[_T]):
    def __init__(self, worker_name: str = "trajectory-writer", max_queue_size: int = 4096, max_batch: int = 1):
        """`max_batch` > 1: tasks that are already waiting are handed to `_process_batch` together (one transaction
        for many rows); the worker never waits to fill a batch."""
        if max_queue_size <= 0:
            raise ValueError("max_queue_size must be positive")
        self._name, self._max, self._max_batch = worker_name, max_queue_size, max(int(max_batch), 1)
        self._q: "queue.Queue" = queue.Queue(maxsize=max_queue_size)
        self._closed = False
        self._lock = threading.Lock()
        self.errors = 0
        self.written = 0
        self._thread = threading.Thread(target=self._worker_loop, name=worker_name, daemon=True)
        self._thread.start()
        _live.add(self)

    @property
    def worker_name(self) -> str:
        return self._name

    @property
    def max_queue_size(self) -> int:
        return self._max

    @property
    def is_closed(self) -> bool:
        return self._closed

    def _enqueue(self, task: _T, timeout: Optional[float] = None) -> None:
        """Blocks while the queue is full (up to `timeout`, then `queue.Full`)."""
        if self._closed:
            raise WriterClosedError(f"{self._name} is closed")
        self._q.put(task, timeout=timeout)

    def _apply(self, tasks: list) -> None:
        if len(tasks) > 1:
            try:
                self._process_batch(tasks)
                self.written += len(tasks)
                return
            except Exception:                                 # find the task that fails: one at a time
                log.warning("%s: a batch of %d tasks failed; retrying them one by one", self._name, len(tasks))
        for t in tasks:
            try:
                self._process_task(t)
                self.written += 1
            except Exception:
                self.errors += 1
                self._log_task_error(t)

    def _worker_loop(self) -> None:
        while True:
            items = [self._q.get()]
            while len(items) < self._max_batch:
                try:
                    items.append(self._q.get_nowait())
                except queue.Empty:
                    break
            tasks: list = []
            stop = False
            try:
                for it in items:
                    if it is _STOP:
                        stop = True
                        break
                    if isinstance(it, threading.Event):       # flush marker: everything before it is applied first
                        if tasks:
                            self._apply(tasks)
                            tasks = []
                        it.set()
                    else:
                        tasks.append(it)
                if tasks:
                    self._apply(tasks)
            finally:
                for _ in items:
                    self._q.task_done()
            if stop:
                return

    def _process_batch(self, tasks: list) -> None:
        """Apply several tasks at once; must be all-or-nothing (the worker retries them singly after a failure)."""
        for t in tasks:
            self._process_task(t)

    @abc.abstractmethod
    def _process_task(self, task: _T) -> None:
        ...

    def _log_task_error(self, task: _T) -> None:
        log.exception("%s: write task failed: %r", self._name, task)

    def flush(self, timeout: Optional[float] = None) -> bool:
        """True when every task queued before the call has been applied."""
        if not self._thread.is_alive():
            return self._q.empty()
        marker = threading.Event()
        self._q.put(marker)
        return marker.wait(timeout)

    def close(self, timeout: Optional[float] = 5.0) -> None:
        with self._lock:
            if self._closed:
                return
            self._closed = True
        self._q.put(_STOP)
        self._thread.join(timeout)
        if self._thread.is_alive():
            log.warning("%s did not stop within %.1f s; %d task(s) may be unwritten", self._name, timeout or 0.0, self._q.qsize())
        _live.discard(self)

    def __del__(self) -> None:
        try:
            self.close(timeout=1.0)
        except Exception:
            pass
