"""Rollout, inference and trainer workers on the worker state machine
(tunix/experimental/worker/{rollout_worker,inference_worker,trainer_worker}.py).

Each wraps an in-process engine behind `AbstractWorker` (checked state transitions, admission limit, heartbeat
reports), speaks the DTOs of `experimental.common.datatypes`, and describes itself with a `WorkerInfo` for the
registry. The transport in front of them (the reference's gRPC actor layer) is not part of this package: the
workers are driven in process."""
from __future__ import annotations

from typing import Any, Callable, Optional, Sequence

import numpy as np

from ..common.datatypes import RolloutRequest, RolloutResponse
from ..common.lineage import LineageContext
from ..orchestrator.worker_registry import WorkerInfo
from .abstract_worker import AbstractWorker


class RolloutWorker(AbstractWorker):
    """Serves `RolloutRequest`s from a generation engine.

    `engine` is either an `EngineServer` (requests join its running batch; weight syncs pause and resume it) or any
    callable `(prompt_token_ids=[...], max_generation_steps=..., temperature=..., top_p=..., top_k=..., seed=...,
    return_logprobs=True)` returning an object with `tokens`, `logprobs`, `text` (the `Sampler` / `PagedEngine`
    call signature). `apply_weights(version, payload)` installs new weights into the engine's model."""

    role = "rollout"

    def __init__(self, worker_id: str, engine, *, apply_weights: Optional[Callable[[int, Any], None]] = None,
                 eos_tokens: Optional[Sequence[int]] = None, max_inflight: int = 64, on_report=None):
        super().__init__(worker_id, max_inflight=max_inflight, on_report=on_report)
        self.engine, self._apply, self.eos_tokens = engine, apply_weights, list(eos_tokens or [])
        self.served = 0

    def info(self) -> WorkerInfo:
        return WorkerInfo(self.worker_id, (self.role,))

    def _initialize(self) -> bool:
        return False

    def _handle(self, req: RolloutRequest) -> RolloutResponse:
        if hasattr(self.engine, "submit"):                      # server mode: one request, own token limit
            toks, lps = self.engine.generate(list(req.prompt_token_ids), req.max_tokens)
            text = None
        else:
            out = self.engine(prompt_token_ids=[list(req.prompt_token_ids)], max_generation_steps=req.max_tokens,
                              temperature=req.temperature, top_p=req.top_p, top_k=req.top_k, seed=req.seed,
                              return_logprobs=True, **({"eos_tokens": self.eos_tokens} if self.eos_tokens else {}))
            toks = np.asarray(out.tokens[0])
            lps = np.asarray(out.logprobs[0], np.float32) if out.logprobs is not None else None
            text = out.text[0] if getattr(out, "text", None) else None
        self.served += 1
        finished = len(toks) > 0 and int(toks[-1]) in self.eos_tokens
        meta = dict(req.metadata)
        lineage = meta.get("lineage")
        if isinstance(lineage, LineageContext):
            lineage.add_event("worker.rollout", "generate", {"worker_id": self.worker_id, "tokens": int(len(toks)),
                                                             "policy_version": self.policy_version})
        return RolloutResponse(req.request_id, [int(t) for t in toks], None if lps is None else [float(x) for x in lps], text,
                               policy_version=self.policy_version, finish_reason="stop" if finished else "length",
                               group_id=req.group_id, metadata=meta)

    def _sync_weights(self, version: int, payload: Any) -> None:
        paused = hasattr(self.engine, "pause") and self.engine.pause(timeout=600)
        try:
            if self._apply is not None:
                self._apply(version, payload)
        finally:
            if paused:
                self.engine.resume()

    def _drain(self) -> None:
        if hasattr(self.engine, "close"):
            self.engine.close()


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
