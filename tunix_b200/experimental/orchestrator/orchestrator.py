"""In-process RL orchestrator over the worker stack (tunix/experimental/orchestrator/{orchestrator,
distributed_rl_engine,rl_program,algorithm_adapter}.py, in miniature).

One training run is a pipeline of the pieces of this package:

  prompts --DispatchWindow--> rollout workers (G generations per prompt, spread over the `rollout` group)
          --> groups of G --AlgorithmAdapter--> rewards, group advantages --> RLTrainerPayload per trajectory
          --BatchAssembler--> micro-batches --> trainer worker `fwd_bwd` ...
          after `rollouts_per_optimizer_update` trajectories: `update`, weight-sync round to every rollout
          worker (its state machine refuses work while SYNCING), `DispatchWindow.release()`.

The transport between the pieces is plain calls and threads; what the reference sends over gRPC goes through the
same DTOs here. A rollout that fails is retried on the next worker of the group and the failed worker is left out."""
from __future__ import annotations

import concurrent.futures as cf
import dataclasses
import itertools
from typing import Any, Callable, Iterable, Optional, Sequence

import numpy as np

from ..common.datatypes import RLTrainerPayload, RolloutRequest, WorkerState
from ..common.lineage import LineageContext
from .batch_assembly import summarize_padding_stats


@dataclasses.dataclass
class AlgorithmAdapter:
    """What differs between algorithms: the reward of a response and the advantages within a prompt's group."""
    reward_fn: Callable[[dict, Any], float]                         # (prompt item, RolloutResponse) -> reward
    advantage_fn: Optional[Callable[[np.ndarray], np.ndarray]] = None
    drop_uniform_groups: bool = True                                # a group whose rewards are all equal teaches nothing

    def advantages(self, rewards: np.ndarray) -> np.ndarray:
        if self.advantage_fn is not None:
            return np.asarray(self.advantage_fn(rewards), np.float32)
        return ((rewards - rewards.mean()) / (rewards.std() + 1e-6)).astype(np.float32)        # GRPO


class Orchestrator:
    def __init__(self, registry, assembler, adapter: AlgorithmAdapter, *, group_size: int, window=None,
                 export_weights: Optional[Callable[[], Any]] = None, rollout_params: Optional[dict] = None,
                 max_threads: int = 16, streaming: bool = False):
        self.registry, self.assembler, self.adapter = registry, assembler, adapter
        self.group_size, self.window = group_size, window
        self.export_weights = export_weights
        self.rollout_params = dict(rollout_params or {})
        self._pool = cf.ThreadPoolExecutor(max_workers=max_threads, thread_name_prefix="orchestrator")
        self._group_pool = cf.ThreadPoolExecutor(max_workers=max(2, max_threads // 2), thread_name_prefix="orchestrator-group")
        self.streaming = streaming
        self._rr = itertools.count()
        self._seed = itertools.count(int(self.rollout_params.pop("seed", None) or 0))     # every generation samples anew
        self.policy_version = 0
        self.history: list = []
        self.excluded: set = set()

    # ------------------------------------------------------------------ rollout
    def _rollout_workers(self) -> list:
        ws = [w for w in self.registry.group("rollout") if w.worker_id not in self.excluded]
        if not ws:
            raise RuntimeError("no rollout worker is left")
        return ws

    def _one_rollout(self, req: RolloutRequest):
        last = None
        for _ in range(len(self._rollout_workers())):
            ws = self._rollout_workers()
            w = ws[next(self._rr) % len(ws)]
            try:
                return w.submit(req)
            except Exception as e:              # the worker's state machine has marked it FAILED
                last = e
                if w.state == WorkerState.FAILED:
                    self.excluded.add(w.worker_id)
        raise RuntimeError(f"rollout {req.request_id} failed on every worker") from last

    def _group(self, step: int, item: dict, seeds: Optional[Sequence[int]] = None) -> list:
        pid = str(item.get("prompt_id", id(item)))
        reqs = []
        seeds = list(seeds) if seeds is not None else [next(self._seed) for _ in range(self.group_size)]
        for g in range(self.group_size):
            lin = LineageContext(tracking_id=f"traj_{pid}_{g}")
            lin.add_event("engine.dispatch", "rollout", {"step": step, "policy_version": self.policy_version})
            reqs.append(RolloutRequest(f"{pid}/{g}", list(item["prompt_ids"]), group_id=pid, policy_version=self.policy_version,
                                       metadata={"lineage": lin}, seed=seeds[g], **self.rollout_params))
        return list(self._pool.map(self._one_rollout, reqs))

    def _payloads(self, item: dict, responses: Sequence) -> list:
        if hasattr(self.adapter, "create_payloads"):        # algorithm_adapter.GRPOAdapter / PPOAdapter
            return self.adapter.create_payloads(item, responses)
        rewards = np.asarray([self.adapter.reward_fn(item, r) for r in responses], np.float32)
        if self.adapter.drop_uniform_groups and float(rewards.std()) == 0.0:
            return []
        adv = self.adapter.advantages(rewards)
        out = []
        for r, a, rew in zip(responses, adv, rewards):
            n = len(r.tokens)
            ex = {"prompt_ids": np.asarray(item["prompt_ids"], np.int32), "completion_ids": np.asarray(r.tokens, np.int32),
                  "completion_mask": np.ones(n, np.float32), "advantages": np.full(n, a, np.float32),
                  "lineage": r.metadata.get("lineage"), "prompt_id": str(item.get("prompt_id", ""))}
            if r.logprobs is not None:
                ex["old_per_token_logps"] = np.asarray(r.logprobs, np.float32)
            out.append(RLTrainerPayload(ex, policy_version=r.policy_version, group_id=r.group_id, reward=float(rew)))
        return out

    # --------------------------------------------------------------------- step
    def _sync_weights(self) -> None:
        self.policy_version += 1
        payload = self.export_weights() if self.export_weights is not None else None
        for w in self._rollout_workers():
            w.sync_weights(self.policy_version, payload)

    def step(self, step: int, prompts: Sequence[dict], streaming: Optional[bool] = None) -> dict:
        """One optimizer update from the given prompts (each rolled out `group_size` times).

        With `streaming` (default: the constructor's setting) the trainer starts on the first micro-batch as soon as
        enough groups have come back to fill it, while the remaining prompts are still being generated: rollout and
        the training passes overlap instead of running one after the other (the reference's streaming gradient
        accumulation, tunix/experimental/orchestrator/rl_program.py). One assembled micro-batch is always held
        back so that the last one can be flagged for the sharded optimizer's gradient reduction."""
        streaming = self.streaming if streaming is None else streaming
        trainer = self.registry.group("trainer").members()[0]
        rewards, stats, losses = [], [], []
        count = {"traj": 0, "filtered": 0, "batches": 0, "overlapped": 0}
        held: list = []

        def train(batch, last: bool) -> None:
            out = trainer.submit({"op": "fwd_bwd", "batch": batch.arrays, "is_last_microbatch": last})
            batch.lineage.add_event("worker.trainer", "fwd_bwd", {"loss": out["loss"], "step": step})
            losses.append(out["loss"])
            stats.append(batch.stats)
            count["batches"] += 1

        def push(batches, rollouts_pending: bool) -> None:
            for b in batches:
                held.append(b)
                if streaming and len(held) > 1:
                    train(held.pop(0), False)
                    count["overlapped"] += int(rollouts_pending)

        def consume(item, responses, rollouts_pending: bool) -> None:
            payloads = self._payloads(item, responses)
            if not payloads:
                count["filtered"] += 1
                if self.window is not None:
                    self.window.on_group_filtered([item])
                return
            rewards.extend(p.reward for p in payloads)
            count["traj"] += len(payloads)
            push(self.assembler.feed(payloads), rollouts_pending)
            if self.window is not None:
                self.window.record_committed_groups([[item]])

        admitted = [it for it in prompts if self.window is None or self.window.admit(it)]
        if streaming:
            # seeds are drawn here, in prompt order, so that a run does not depend on which group a thread picks up first
            futs = {self._group_pool.submit(self._group, step, it, [next(self._seed) for _ in range(self.group_size)]): it
                    for it in admitted}
            left = len(futs)
            for f in cf.as_completed(futs):
                left -= 1
                consume(futs[f], f.result(), left > 0)
        else:
            for it in admitted:
                consume(it, self._group(step, it), False)
        push(self.assembler.flush(), False)
        while held:
            train(held.pop(0), len(held) == 0)
        rec = {"step": step, "trajectories": count["traj"], "filtered_groups": count["filtered"], "microbatches": count["batches"],
               "reward_mean": float(np.mean(rewards)) if rewards else 0.0, "loss": float(np.mean(losses)) if losses else None}
        if streaming:
            rec["microbatches_overlapped_with_rollout"] = count["overlapped"]
        if count["batches"]:
            up = trainer.submit({"op": "update"})
            rec.update(grad_norm=up["grad_norm"], train_step=up["step"], **summarize_padding_stats(stats))
            self._sync_weights()
        rec["policy_version"] = self.policy_version
        if self.window is not None:
            self.window.release()
        self.history.append(rec)
        return rec

    def run(self, prompt_batches: Iterable[Sequence[dict]], max_steps: Optional[int] = None) -> list:
        for step, prompts in enumerate(prompt_batches):
            if max_steps is not None and step >= max_steps:
                break
            self.step(step, prompts)
        return self.history

    def close(self) -> None:
        self._pool.shutdown(wait=False, cancel_futures=True)
        self._group_pool.shutdown(wait=False, cancel_futures=True)
