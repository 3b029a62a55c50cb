"""The single-call rollout worker on the worker state machine (tunix/experimental/worker/rollout_worker.py).

It wraps a generation engine behind `AbstractWorker` (checked state transitions, admission limit, heartbeat
reports), speaks the DTOs of `experimental.common.datatypes`, and describes itself with a `WorkerInfo` for the
registry. `inference_worker.InferenceWorker` and `trainer_worker.TrainerWorker` are its siblings (also importable from
here); `agentic_rollout_worker.AgenticRolloutWorker` runs whole episodes; `remote_execution` puts any of them behind
gRPC."""
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


def __getattr__(name):
    """`InferenceWorker` and `TrainerWorker` used to live in this module; they are still importable from it."""
    if name == "InferenceWorker":
        from .inference_worker import InferenceWorker
        return InferenceWorker
    if name == "TrainerWorker":
        from .trainer_worker import TrainerWorker
        return TrainerWorker
    raise AttributeError(name)
