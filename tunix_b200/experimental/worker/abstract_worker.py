"""Worker lifecycle (tunix/experimental/worker/abstract_worker.py): a state machine with checked transitions,
heartbeat reports and admission control; concrete workers fill in `_initialize`, `_handle`, `_sync_weights`."""
from __future__ import annotations

import abc
import threading
from typing import Any, Callable, Optional

from ..common.datatypes import HealthReport, WorkerState, check_transition


class AbstractWorker(abc.ABC):
    def __init__(self, worker_id: str, max_inflight: int = 1, on_report: Optional[Callable[[HealthReport], None]] = None):
        self.worker_id, self.max_inflight = worker_id, max_inflight
        self._state = WorkerState.CREATED
        self._lock = threading.RLock()
        self._inflight = 0
        self.policy_version = 0
        self._on_report = on_report
        self.last_error: Optional[BaseException] = None

    # ---------------------------------------------------------------- state
    @property
    def state(self) -> WorkerState:
        return self._state

    def _set(self, new: WorkerState, detail: str = "") -> None:
        with self._lock:
            check_transition(self._state, new)
            self._state = new
        self.report(detail)

    def report(self, detail: str = "") -> HealthReport:
        r = HealthReport(self.worker_id, self._state, policy_version=self.policy_version, inflight=self._inflight, detail=detail)
        if self._on_report:
            self._on_report(r)
        return r

    # ------------------------------------------------------------ lifecycle
    def start(self) -> None:
        self._set(WorkerState.INITIALIZING)
        try:
            needs_compile = self._initialize()
            if needs_compile:
                self._set(WorkerState.COMPILING)
                self._compile()
            self._set(WorkerState.READY)
        except BaseException as e:
            self._fail(e)
            raise

    def submit(self, request: Any) -> Any:
        with self._lock:
            if self._state not in (WorkerState.READY, WorkerState.BUSY):
                raise RuntimeError(f"{self.worker_id} is {self._state.value}; it does not take work")
            if self._inflight >= self.max_inflight:
                raise RuntimeError(f"{self.worker_id} is at its admission limit ({self.max_inflight})")
            self._inflight += 1
            if self._state == WorkerState.READY:
                self._set(WorkerState.BUSY)
        try:
            return self._handle(request)
        except BaseException as e:
            self._fail(e)
            raise
        finally:
            with self._lock:
                self._inflight -= 1
                if self._inflight == 0 and self._state == WorkerState.BUSY:
                    self._set(WorkerState.READY)

    def sync_weights(self, version: int, payload: Any = None) -> None:
        self._set(WorkerState.SYNCING, f"to version {version}")
        try:
            self._sync_weights(version, payload)
            self.policy_version = version
            self._set(WorkerState.READY)
        except BaseException as e:
            self._fail(e)
            raise

    def stop(self) -> None:
        if self._state in (WorkerState.STOPPED,):
            return
        if self._state == WorkerState.FAILED:
            self._set(WorkerState.STOPPED)
            return
        if self._state in (WorkerState.READY, WorkerState.BUSY):
            self._set(WorkerState.DRAINING)
            self._drain()
        self._set(WorkerState.STOPPED) if self._state == WorkerState.DRAINING else None

    def _fail(self, e: BaseException) -> None:
        self.last_error = e
        with self._lock:
            if self._state not in (WorkerState.FAILED, WorkerState.STOPPED):
                self._state = WorkerState.FAILED
        self.report(repr(e))

    # ---------------------------------------------------------------- hooks
    @abc.abstractmethod
    def _initialize(self) -> bool:
        """Returns True when a compile / graph-capture phase follows."""

    def _compile(self) -> None:
        pass

    @abc.abstractmethod
    def _handle(self, request: Any) -> Any: ...

    def _sync_weights(self, version: int, payload: Any) -> None:
        pass

    def _drain(self) -> None:
        pass
