"""Admission control of a rollout worker (tunix/experimental/worker/traffic_controller.py:29-153).

One object owns the worker's serving state and the set of request tasks in flight, so that a weight sync can
close the gate, wait for the running requests and reopen, without locks spread over worker and manager:

  READY --close_for_sync()--> SYNCING --reopen()--> READY        stop() from anywhere --> STOPPED (final)

Tasks live on the event loop the controller was created on; every method may be called from other threads."""
from __future__ import annotations

import asyncio
import threading
from typing import Any

from ..common.datatypes import WorkerState


class AdmissionClosedError(RuntimeError):
    """A request arrived while the gate is closed for a weight sync or after the worker stopped."""


class TrafficController:
    def __init__(self, loop: asyncio.AbstractEventLoop | None = None):
        self._loop = loop or asyncio.get_running_loop()
        self._lock = threading.RLock()
        self._state = WorkerState.READY
        self._open = asyncio.Event()
        self._on_loop(self._open.set)
        self._tasks: set = set()

    def _on_loop(self, fn, loop=None) -> None:
        loop = loop or self._loop
        try:
            here = asyncio.get_running_loop()
        except RuntimeError:
            here = None
        fn() if here is loop else loop.call_soon_threadsafe(fn)

    @property
    def state(self) -> WorkerState:
        with self._lock:
            return self._state

    def is_admission_open(self) -> bool:
        with self._lock:
            return self._state == WorkerState.READY

    async def wait_for_admission(self) -> None:
        await self._open.wait()

    def try_admit(self, task: "asyncio.Task[Any]") -> bool:
        """Track the task when the worker is READY; otherwise cancel it and return False."""
        with self._lock:
            if self._state != WorkerState.READY:
                self._on_loop(task.cancel, task.get_loop())
                return False
            self._tasks.add(task)
        task.add_done_callback(self._done)
        return True

    def _done(self, task) -> None:
        with self._lock:
            self._tasks.discard(task)

    def active_tasks(self) -> list:
        with self._lock:
            return list(self._tasks)

    async def drain(self, timeout_s: float | None = None) -> bool:
        """Wait for the tracked tasks; True when none is left."""
        tasks = self.active_tasks()
        if tasks:
            await asyncio.wait(tasks, timeout=timeout_s)
        return not self.active_tasks()

    def close_for_sync(self) -> None:
        with self._lock:
            if self._state not in (WorkerState.READY, WorkerState.SYNCING):
                raise RuntimeError(f"cannot start a weight sync from {self._state.value}")
            self._state = WorkerState.SYNCING
            self._on_loop(self._open.clear)

    def reopen(self) -> bool:
        with self._lock:
            if self._state == WorkerState.STOPPED:
                return False
            self._state = WorkerState.READY
            self._on_loop(self._open.set)
            return True

    def stop(self) -> list:
        """Final: closes the gate and cancels what is running. Returns the cancelled tasks."""
        with self._lock:
            self._state = WorkerState.STOPPED
            self._on_loop(self._open.clear)
            tasks = list(self._tasks)
        for t in tasks:
            self._on_loop(t.cancel, t.get_loop())
        return tasks
