"""A worker whose behaviour is scripted, for control-plane tests (tunix/experimental/worker/mock_worker.py)."""
from __future__ import annotations

import time
from typing import Any, Callable, Optional

from .abstract_worker import AbstractWorker


class MockWorker(AbstractWorker):
    def __init__(self, worker_id: str, handler: Optional[Callable[[Any], Any]] = None, latency_s: float = 0.0,
                 fail_on_init: bool = False, fail_on_sync: bool = False, needs_compile: bool = False, **kw):
        super().__init__(worker_id, **kw)
        self.handler, self.latency_s = handler or (lambda r: r), latency_s
        self.fail_on_init, self.fail_on_sync, self.needs_compile = fail_on_init, fail_on_sync, needs_compile
        self.handled: list = []

    def _initialize(self) -> bool:
        if self.fail_on_init:
            raise RuntimeError("scripted initialisation failure")
        return self.needs_compile

    def _handle(self, request):
        if self.latency_s:
            time.sleep(self.latency_s)
        self.handled.append(request)
        return self.handler(request)

    def _sync_weights(self, version, payload):
        if self.fail_on_sync:
            raise RuntimeError("scripted weight-sync failure")

    def info(self):
        from ..orchestrator.worker_registry import WorkerInfo
        return WorkerInfo(self.worker_id, (getattr(self, "role", "mock"),))


def make_echo_worker(worker_id: str, role: str = "rollout", scale: int = 1, latency_s: float = 0.0) -> MockWorker:
    """Factory for process-launch tests and demos: answers a request `x` with `x * scale`."""
    w = MockWorker(worker_id, handler=lambda r: r * scale, latency_s=latency_s)
    w.role = role
    return w
