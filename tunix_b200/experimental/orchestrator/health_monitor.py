"""Heartbeat bookkeeping with per-state deadlines (tunix/experimental/orchestrator/health_monitor.py:36-176).

Workers push `HealthReport`s; `check()` names the workers that are unhealthy: silent for longer than the
heartbeat timeout, or sitting in a transitional state (COMPILING 30 min, SYNCING 10 min, DRAINING 5 min) longer
than that state's deadline. The clock is injectable so tests can move time by hand."""
from __future__ import annotations

import dataclasses
import threading
import time
from typing import Callable, Optional

from ..common.datatypes import HealthReport, WorkerState

STATE_DEADLINES_S = {WorkerState.COMPILING: 30 * 60.0, WorkerState.SYNCING: 10 * 60.0, WorkerState.DRAINING: 5 * 60.0,
                     WorkerState.INITIALIZING: 10 * 60.0}


@dataclasses.dataclass
class Unhealthy:
    worker_id: str
    reason: str          # "heartbeat" | "state_deadline" | "failed"
    state: WorkerState
    seconds: float


class HealthMonitor:
    def __init__(self, heartbeat_timeout_s: float = 60.0, state_deadlines: Optional[dict] = None,
                 clock: Callable[[], float] = time.monotonic):
        self.heartbeat_timeout_s = heartbeat_timeout_s
        self.deadlines = dict(STATE_DEADLINES_S, **(state_deadlines or {}))
        self.clock = clock
        self._lock = threading.Lock()
        self._last_seen: dict = {}
        self._state: dict = {}
        self._state_since: dict = {}

    def observe(self, report: HealthReport) -> None:
        now = self.clock()
        with self._lock:
            wid = report.worker_id
            self._last_seen[wid] = now
            if self._state.get(wid) != report.state:
                self._state[wid], self._state_since[wid] = report.state, now

    def forget(self, worker_id: str) -> None:
        with self._lock:
            for d in (self._last_seen, self._state, self._state_since):
                d.pop(worker_id, None)

    def check(self) -> list:
        now = self.clock()
        out = []
        with self._lock:
            for wid, seen in self._last_seen.items():
                st = self._state[wid]
                if st == WorkerState.STOPPED:
                    continue
                if st == WorkerState.FAILED:
                    out.append(Unhealthy(wid, "failed", st, now - self._state_since[wid]))
                elif now - seen > self.heartbeat_timeout_s:
                    out.append(Unhealthy(wid, "heartbeat", st, now - seen))
                elif st in self.deadlines and now - self._state_since[wid] > self.deadlines[st]:
                    out.append(Unhealthy(wid, "state_deadline", st, now - self._state_since[wid]))
        return out

    def healthy_workers(self) -> list:
        bad = {u.worker_id for u in self.check()}
        with self._lock:
            return sorted(w for w, s in self._state.items() if w not in bad and s in (WorkerState.READY, WorkerState.BUSY))
