"""The scoring worker (tunix/experimental/worker/inference_worker.py): a frozen model behind the worker state machine."""
from __future__ import annotations

from typing import Any

from ..orchestrator.worker_registry import WorkerInfo
from .abstract_worker import AbstractWorker


class InferenceWorker(AbstractWorker):
    """Scores sequences with a frozen model (reference / old-policy log-probs, values, rewards). `score_fns` maps
    an operation name to `fn(**arrays) -> array`; a request is `{"op": name, **arrays}`."""

    role = "inference"

    def __init__(self, worker_id: str, score_fns: dict, *, apply_weights=None, max_inflight: int = 4, on_report=None):
        super().__init__(worker_id, max_inflight=max_inflight, on_report=on_report)
        self.score_fns, self._apply = dict(score_fns), apply_weights

    def info(self) -> WorkerInfo:
        return WorkerInfo(self.worker_id, (self.role,), attributes={"ops": sorted(self.score_fns)})

    def _initialize(self) -> bool:
        return False

    def _handle(self, req: dict):
        req = dict(req)
        op = req.pop("op")
        if op not in self.score_fns:
            raise KeyError(f"{self.worker_id} has no operation {op!r}; known: {sorted(self.score_fns)}")
        return self.score_fns[op](**req)

    def _sync_weights(self, version: int, payload: Any) -> None:
        if self._apply is not None:
            self._apply(version, payload)
