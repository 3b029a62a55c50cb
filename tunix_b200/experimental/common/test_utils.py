"""Stand-ins for the workers of the distributed stack (tunix/experimental/common/test_utils.py): enough behaviour to
exercise an engine, a program or an algorithm adapter on a laptop, with no model and no GPU, and with failures that a
test can switch on from the host.

    eng = DistributedRLEngine([EchoRolloutWorker("r0"), EchoRolloutWorker("r1")], {"actor": RecordingTrainerWorker()})
    StandardRLProgram(GRPOAdapter(reward_fn=token_sum_reward), make_prompts(8), 2, num_generations=4, batch_size=2, ...).run(eng)
"""
from __future__ import annotations

import time
from typing import Any, Callable, Optional

import numpy as np

from .datatypes import RolloutRequest, RolloutResponse


def make_prompts(n: int, seed: int = 0, prompt_len: int = 5, vocab: int = 60) -> list:
    """`n` prompt items `{"prompt_id": "p<i>", "prompt_ids": [...]}` with reproducible token ids."""
    rng = np.random.default_rng(seed)
    return [{"prompt_id": f"p{i}", "prompt_ids": [1] + rng.integers(3, vocab, prompt_len - 1).tolist()} for i in range(n)]


def token_sum_reward(item: dict, response) -> float:
    """A reward that differs between the generations of a prompt: the sum of the response's token ids modulo 5."""
    return float(sum(int(t) % 5 for t in response.tokens))


class EchoRolloutWorker:
    """Answers a request with `n` tokens drawn from the request's seed (so the generations of a prompt differ and a
    re-run repeats them). `fail=True` makes every request raise; `latency_s` (a number or `fn(request) -> seconds`)
    delays it; `transform(request, response)` may rewrite a response; weight syncs are recorded in `synced`."""

    def __init__(self, worker_id: str, *, n: int = 4, vocab: int = 60, fail: bool = False, latency_s: Any = 0.0,
                 transform: Optional[Callable[[RolloutRequest, RolloutResponse], RolloutResponse]] = None):
        self.worker_id, self.n, self.vocab, self.fail, self.latency_s, self.transform = worker_id, n, vocab, fail, latency_s, transform
        self.seen: list = []
        self.synced: list = []
        self.policy_version = 0

    def submit(self, req: RolloutRequest) -> RolloutResponse:
        if self.fail:
            raise ConnectionError(f"{self.worker_id} lost")
        delay = self.latency_s(req) if callable(self.latency_s) else self.latency_s
        if delay:
            time.sleep(float(delay))
        self.seen.append(req)
        toks = np.random.default_rng(req.seed).integers(3, self.vocab, min(self.n, req.max_tokens)).tolist()
        out = RolloutResponse(req.request_id, toks, [-0.5] * len(toks), None, policy_version=self.policy_version, group_id=req.group_id,
                              metadata=dict(req.metadata))
        return self.transform(req, out) if self.transform is not None else out

    def sync_weights(self, version: int, payload: Any = None) -> None:
        self.policy_version = version
        self.synced.append((version, payload))


class RecordingTrainerWorker:
    """Speaks the split-step protocol (`fwd_bwd`, `update`, `save_checkpoint`, `restore_checkpoint`, `get_metrics`),
    records every operation in `ops` as (name, is_last_microbatch) and every micro-batch in `batches`, and keeps its
    "checkpoint" in the dict it is given, so that a second instance over the same dict resumes."""

    def __init__(self, disk: Optional[dict] = None, fail_on: Optional[str] = None):
        self.disk = disk if disk is not None else {}
        self.fail_on = fail_on
        self.ops: list = []
        self.batches: list = []
        self.steps = self.pending = 0

    def submit(self, req: dict):
        req = dict(req)
        op = req.pop("op")
        if op == self.fail_on:
            raise RuntimeError(f"trainer failed in {op}")
        self.ops.append((op, req.get("is_last_microbatch")))
        if op == "fwd_bwd":
            self.pending += 1
            self.batches.append(req.get("batch"))
            return {"loss": 1.0 / (1 + self.steps), "pending_microbatches": self.pending}
        if op == "update":
            if self.pending == 0:
                raise RuntimeError("update() without a preceding fwd_bwd()")
            self.steps, self.pending = self.steps + 1, 0
            return {"step": self.steps, "grad_norm": 1.0}
        if op == "save_checkpoint":
            self.disk["latest"] = dict(req["custom_metadata"])
            return True
        if op == "restore_checkpoint":
            meta = self.disk.get("latest")
            self.steps = int(meta["step"]) if meta and str(meta.get("step", "")).isdigit() else 0
            return dict(meta) if meta else 0
        if op == "get_metrics":
            return {"train_steps": self.steps, "pending_microbatches": self.pending}
        if op == "fwd_only":
            return np.zeros(np.asarray(req["batch"]["input_tokens"]).shape, np.float32)
        raise KeyError(op)


class ConstantInferenceWorker:
    """An inference worker whose every operation answers with a constant of the input's shape (`calls` counts them)."""

    def __init__(self, value: float = -2.0):
        self.value, self.calls = value, 0

    def submit(self, req: dict):
        self.calls += 1
        ref = req.get("input_tokens", req.get("items"))
        return np.full(np.asarray(ref).shape, self.value, np.float32)
