"""The trainer worker (tunix/experimental/worker/trainer_worker.py): the split-step trainer behind the worker state machine."""
from __future__ import annotations

from ..orchestrator.worker_registry import WorkerInfo
from .abstract_worker import AbstractWorker


class TrainerWorker(AbstractWorker):
    """Drives a trainer through the split-step protocol of the distributed engine: `fwd_bwd` on a micro-batch
    (gradients accumulate), `update` (optimizer step, version + 1), `eval_step`, `fwd_only`, `save_checkpoint`,
    `restore_checkpoint`. `trainer` is a `TrainerV2` (`experimental.train.peft_trainer_v2`)."""

    role = "trainer"

    def __init__(self, worker_id: str, trainer, on_report=None):
        super().__init__(worker_id, max_inflight=1, on_report=on_report)
        self.trainer = trainer

    def info(self) -> WorkerInfo:
        return WorkerInfo(self.worker_id, (self.role,))

    def _initialize(self) -> bool:
        return False

    def _handle(self, req: dict):
        req = dict(req)
        op = req.pop("op")
        if op not in ("fwd_bwd", "update", "eval_step", "fwd_only", "save_checkpoint", "restore_checkpoint", "restored_metadata",
                      "get_metrics"):
            raise KeyError(f"unknown trainer operation {op!r}")
        out = getattr(self.trainer, op)(**req)
        if op == "update":
            self.policy_version += 1
        return out

    def _drain(self) -> None:
        """A stopping worker leaves no checkpoint half written: background saves are waited for."""
        wait = getattr(self.trainer, "wait_for_checkpoints", None)
        if wait is not None:
            wait()
