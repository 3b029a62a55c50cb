"""An RL training run as four overlapping stages over an `AbstractRLEngine`
(tunix/experimental/orchestrator/rl_program.py:223-1663).

  dispatch   walks the prompt dataset (prefetched on a thread), waits at the `DispatchWindow` until the batch of a
             prompt is at most `max_staleness` batches ahead of the one the trainer consumes next, stamps the prompt's
             dataset coordinates (`prompt_idx`, `batch_idx`, `intra_batch_idx`) and dispatches G generations;
  polling    collects finished rollouts, groups them by prompt; a full group moves on, a group that is older than
             `max_staleness` policy versions is dropped and reported to the window (a replacement gets dispatched);
  critique   turns a group into trainer payloads through the algorithm adapter (rewards, advantages); rollouts that
             failed are left out, a group that teaches nothing (no payloads) counts as filtered;
  train      one optimizer step per `batch_size` scored groups: payloads go through the batch assembler, every
             assembled micro-batch is handed to `engine.train_step` while the next one is being assembled (one call in
             flight; the last micro-batch of the step is held back so that it can carry `apply_optimizer=True`), then
             checkpoint, weight sync, commit of the consumed prompt ids, metrics, `window.release()`.

Resume: the engine restores the trainer and reports the step; the program continues from that step, with the policy
version the checkpoint recorded, and either skips exactly the prompt ids the checkpoint lists as trained-on or skipped
(off-policy runs) or the dataset prefix that the finished steps consumed.
"""
from __future__ import annotations

import abc
import asyncio
import contextlib
import dataclasses
import logging
import time
from typing import Any, Callable, Iterable, Mapping, Optional

import numpy as np

from ..common.datatypes import GenerationArgs, Role
from ..common.dispatch_window import DispatchWindow
from ..common.logging_utils import summarize_list
from ..common.tagging import prompt_coordinates, tag_prompt
from . import dataset_utils
from .batch_assembly import BatchConfig, create_batch_assembler, summarize_padding_stats

log = logging.getLogger(__name__)
_EOF = object()


def _generation_metrics(groups) -> dict:
    """`rollout/completions/*` of a step from the `raw_length` / `clipped` facts the rollout side recorded; the two
    means are per prompt group, so a short group weighs as much as a full one."""
    clip, mean_len, lengths = [], [], []
    for group in groups:
        ls, clipped = [], 0
        for r in group:
            md = getattr(r, "metadata", None) or {}
            if md.get("clipped") is None or md.get("raw_length") is None:
                continue
            ls.append(int(md["raw_length"]))
            clipped += int(md["clipped"])
        if ls:
            clip.append(clipped / len(ls))
            mean_len.append(float(np.mean(ls)))
            lengths.extend(ls)
    if not lengths:
        return {}
    return {"rollout/completions/clip_ratio": float(np.mean(clip)), "rollout/completions/mean_raw_length": float(np.mean(mean_len)),
            "rollout/completions/max_raw_length": float(np.max(lengths)), "rollout/completions/min_raw_length": float(np.min(lengths))}


@dataclasses.dataclass(kw_only=True)
class RLStepResult:
    step: int
    policy_version: int
    num_rollouts: int
    num_microbatches: int
    reward_mean: float
    reward_std: float
    advantage_mean: float = 0.0
    advantage_std: float = 0.0
    filtered_groups: int = 0
    step_time_s: float = 0.0
    train_result: Any = None


class RLProgram(abc.ABC):
    def __init__(self):
        self._step = 0
        self.policy_version = 0
        self.last_step_result: Optional[RLStepResult] = None
        self.engine = None

    @property
    def step(self) -> int:
        return self._step

    @abc.abstractmethod
    def run(self, engine, **kwargs) -> None:
        ...

    def close(self) -> None:
        pass


@dataclasses.dataclass
class _Group:
    item: dict
    responses: list
    payloads: list = dataclasses.field(default_factory=list)

    @property
    def prompt_id(self) -> str:
        return str(self.item["prompt_id"])

    def __getitem__(self, i):                 # `DispatchWindow` reads the prompt id off the first element of a group
        return (self.item,)[i]

    def __len__(self) -> int:
        return 1


class StandardRLProgram(RLProgram):
    """`algo`: an algorithm adapter (`create_payloads(prompt item, responses) -> [RLTrainerPayload]`;
    `algorithm_adapter.GRPOAdapter` / `PPOAdapter`). `dataset`: an iterable of prompt dicts with `prompt_ids` (token
    ids) and optionally `prompt_id`. `batch_size`: prompt groups per optimizer step. `metrics_logger`: anything with
    `log(prefix, name, value, mode, step)` (`sft.metrics_logger.MetricsLogger`)."""

    def __init__(self, algo, dataset: Optional[Iterable[Any]] = None, max_steps: Optional[int] = None, *, num_generations: int,
                 batch_size: int = 1, assembler=None, batch_config: Optional[BatchConfig] = None, packed: bool = True,
                 generation_args: Optional[GenerationArgs] = None, max_response_length: Optional[int] = None,
                 max_staleness: int = 0, sync_weights: bool = True, checkpoint_every: int = 1, metrics_logger=None,
                 trajectory_store=None, metrics_prefix: str = "", poll_timeout_s: float = 0.2, reference_kl: bool = False,
                 group_order: str = "completion", trajectory_log_dir: Optional[str] = None, mode: str = "train",
                 on_step_begin: Optional[Callable[[int], None]] = None, on_step_end: Optional[Callable[[int, Any], None]] = None):
        super().__init__()
        if max_staleness < 0:
            raise ValueError("max_staleness must be non-negative.")
        if num_generations <= 0 or batch_size <= 0:
            raise ValueError("num_generations and batch_size must be positive.")
        if checkpoint_every < 0:
            raise ValueError("checkpoint_every must be non-negative (0 = never).")
        self.algo, self.dataset, self.max_steps = algo, dataset, max_steps
        self.num_generations, self.full_batch_size = num_generations, batch_size
        self.batch_size = batch_size
        self.generation_args = generation_args or GenerationArgs()
        self.max_response_length = max_response_length
        self.assembler = assembler if assembler is not None else create_batch_assembler(batch_config or BatchConfig(), packed=packed)
        self.max_staleness, self.sync_weights, self.checkpoint_every = max_staleness, sync_weights, checkpoint_every
        self.metrics_logger, self.metrics_prefix = metrics_logger, metrics_prefix
        self._trajectory_store = trajectory_store          # used, not owned: whoever built it closes it
        # one JSON line per consumed rollout (prompt id, group index, reward, versions, tokens), written by a thread
        self.trajectory_logger = None
        if trajectory_log_dir:
            from ...utils.trajectory_logger import AsyncTrajectoryLogger
            self.trajectory_logger = AsyncTrajectoryLogger(trajectory_log_dir)
        self.poll_timeout_s = poll_timeout_s
        # "completion": the trainer takes groups as they finish (best utilisation). "prompt_arrival": groups reach the
        # trainer in the order their prompts were dispatched, whatever order they finished in, so that a run does not
        # depend on rollout timing (a filtered group gives up its place)
        if group_order not in ("completion", "prompt_arrival"):
            raise ValueError(f"group_order must be 'completion' or 'prompt_arrival', got {group_order!r}")
        self.group_order = group_order
        self._order_next, self._order_pending = 0, {}
        # "eval": rollouts are generated, scored and reported step by step (rewards, lengths, staleness), but nothing is
        # assembled, trained, synchronised or checkpointed, and no checkpoint is restored
        if mode not in ("train", "eval"):
            raise ValueError(f"mode must be 'train' or 'eval', got {mode!r}")
        self.mode = mode
        # reference log-probs for a KL term: asked of the REFERENCE role per assembled micro-batch (dense rows: one
        # forward pass over what the trainer will see), stored in the batch as `ref_per_token_logps`
        self.reference_kl = bool(reference_kl or getattr(algo, "requires_reference_kl", False))
        self.on_step_begin, self.on_step_end = on_step_begin, on_step_end
        self.dispatch_window = DispatchWindow(max_staleness, lambda: self._step, full_batch_size=batch_size, out_of_order_resume=True)
        self.history: list = []
        self._in_flight = 0
        self._dispatched = 0
        self._base_step = 0
        self._filtered_groups: list = []
        self._prompts: dict = {}

    @property
    def trajectory_store(self):
        return self._trajectory_store

    def close(self) -> None:
        if self.trajectory_logger is not None:
            self.trajectory_logger.stop()
        if self.metrics_logger is not None and hasattr(self.metrics_logger, "close"):
            self.metrics_logger.close()

    # ------------------------------------------------------------------ resume
    async def _resume_from_checkpoint(self) -> None:
        restored = await self.engine.resume_from_checkpoint(role=Role.ACTOR, resync_rollout_weights=self.sync_weights)
        step = restored[0] if isinstance(restored, tuple) else restored
        if not step or step <= 0:
            return
        self._step = self.policy_version = int(step)
        meta = self.engine.restored_checkpoint_metadata
        if isinstance(meta, Mapping) and meta.get("policy_version") is not None and (
                "committed_prompt_ids" in meta or "skipped_prompt_ids" in meta):
            self.policy_version = int(meta["policy_version"])
        if self.dispatch_window.restore_checkpoint_metadata(meta):
            log.info("resuming an off-policy run: step=%d policy_version=%d (%d prompts trained on, %d skipped)", step,
                     self.policy_version, len(self.dispatch_window.committed_prompt_ids), len(self.dispatch_window.skipped_prompt_ids))
        else:
            log.info("resuming: step=%d policy_version=%d, skipping %d dataset items", step, self.policy_version,
                     self.dispatch_window.dataset_skip_count)

    # ------------------------------------------------------------------ stage 1a: dispatch
    async def rollout_dispatch_stage(self) -> None:
        if self.dataset is None:
            raise ValueError("StandardRLProgram needs a dataset, at construction or in run().")
        try:
            async for idx, item in dataset_utils.iter_dataset_async(self.dataset, skip_count=self.dispatch_window.dataset_skip_count,
                                                                    prefetch_size=max(1, self.full_batch_size)):
                if not isinstance(item, Mapping):
                    item = {"prompt_ids": item}
                item = dict(item)
                item.setdefault("prompt_id", f"prompt_{idx}")
                if not self.dispatch_window.admit(item):
                    continue
                # the window counts admitted prompts of this run, not dataset positions: after a resume by prompt id the
                # two differ (prompts the earlier run trained on or skipped are passed over above)
                await self.dispatch_window.wait_for(self._base_step + self._dispatched // self.full_batch_size)
                if self.max_response_length is not None:
                    item.setdefault("max_response_length", self.max_response_length)
                item = tag_prompt(item, {**prompt_coordinates(idx, self.full_batch_size), "dispatch_seq": self._dispatched})
                self._prompts[str(item["prompt_id"])] = item
                self._in_flight += self.num_generations
                self._dispatched += 1
                await self.engine.dispatch_rollouts([item], num_generations=self.num_generations, policy_version=self.policy_version,
                                                    generation_args=self.generation_args)
        finally:
            self._dispatch_done.set()

    # ------------------------------------------------------------------ stage 1b: polling
    def _filter_group(self, group: _Group, why: str) -> None:
        log.info("[pipeline] FILTERED prompt_id=%s (%s)", group.prompt_id, why)
        self._filtered_groups.append((group.prompt_id, why))
        self._prompts.pop(group.prompt_id, None)
        self.dispatch_window.on_group_filtered(group)
        self._hand_to_trainer(group, None)

    def _hand_to_trainer(self, group: _Group, scored: Optional[_Group]) -> None:
        """Queue a scored group for the train stage (`scored` None: the group was filtered and only gives up its place)."""
        if self.group_order == "completion":
            if scored is not None:
                self._scored_q.put_nowait(scored)
            return
        seq = (group.item.get("metadata") or {}).get("dispatch_seq")
        if seq is None:                                   # not dispatched by this program: no place to keep
            if scored is not None:
                self._scored_q.put_nowait(scored)
            return
        self._order_pending[int(seq)] = scored
        while self._order_next in self._order_pending:
            g = self._order_pending.pop(self._order_next)
            self._order_next += 1
            if g is not None:
                self._scored_q.put_nowait(g)

    def _flush_order(self) -> None:
        """End of the dataset: what is still held goes out in order (places of groups that never completed stay empty)."""
        for seq in sorted(self._order_pending):
            g = self._order_pending.pop(seq)
            if g is not None:
                self._scored_q.put_nowait(g)

    async def polling_stage(self) -> None:
        open_groups: dict = {}
        try:
            while not self._dispatch_done.is_set() or self._in_flight > 0:
                try:
                    completed = await self.engine.poll_rollouts(timeout_s=self.poll_timeout_s)
                except Exception as e:
                    log.warning("polling failed: %s", e)
                    await asyncio.sleep(0.01)
                    continue
                if not completed:
                    await asyncio.sleep(0.002)          # an engine that answers at once must not turn this loop into a spin
                    continue
                self._in_flight -= len(completed)
                for r in completed:
                    pid = str(r.group_id)
                    bucket = open_groups.setdefault(pid, [])
                    bucket.append(r)
                    if len(bucket) < self.num_generations:
                        continue
                    del open_groups[pid]
                    bucket.sort(key=lambda x: (x.metadata or {}).get("group_index", 0))
                    group = _Group(self._prompts.get(pid) or {"prompt_id": pid}, bucket)
                    oldest = min(int(x.policy_version) for x in bucket)
                    if self.policy_version - oldest > self.max_staleness:
                        self._filter_group(group, f"stale: policy_version {oldest} < {self.policy_version} - {self.max_staleness}")
                        continue
                    await self._raw_q.put(group)
            if open_groups:
                log.warning("dropping %d incomplete prompt group(s) at the end of the dataset", len(open_groups))
        finally:
            await self._raw_q.put(_EOF)

    # ------------------------------------------------------------------ stage 2: critique
    async def critique_stage(self) -> None:
        try:
            while True:
                group = await self._raw_q.get()
                if group is _EOF:
                    break
                valid = [r for r in group.responses if (r.metadata or {}).get("is_valid", True) and len(r.tokens) > 0]
                if len(valid) < min(2, self.num_generations):
                    self._filter_group(group, "too few valid rollouts")
                    continue
                payloads = await asyncio.to_thread(self.algo.create_payloads, group.item, valid)
                if not payloads:
                    self._filter_group(group, "no learning signal")
                    continue
                group.payloads, group.responses = list(payloads), valid        # payload i belongs to response i from here on
                log.info("[pipeline] ARRIVED prompt_id=%s batch_idx=%s policy_version=%d", group.prompt_id,
                         (group.item.get("metadata") or {}).get("batch_idx"), int(valid[0].policy_version))
                self._hand_to_trainer(group, group)
        finally:
            self._flush_order()
            await self._scored_q.put(_EOF)

    # ------------------------------------------------------------------ stage 3: train
    def _log_metric(self, name: str, value, step: int) -> None:
        if self.metrics_logger is None or value is None:
            return
        prefix, _, leaf = name.rpartition("/")
        prefix = prefix or "global"
        if self.metrics_prefix:
            prefix = f"{self.metrics_prefix}/{prefix}"
        from ...sft.metrics_logger import Mode
        self.metrics_logger.log(prefix, leaf, value, Mode.TRAIN if self.mode == "train" else Mode.EVAL, step)

    def _store_trajectories(self, groups, step: int) -> None:
        if self.trajectory_logger is not None:
            for g in groups:
                for p, r in zip(g.payloads, g.responses):
                    self.trajectory_logger.log({"step": step, "prompt_id": g.prompt_id, "request_id": r.request_id,
                                                "group_index": (r.metadata or {}).get("group_index"), "reward": float(p.reward or 0.0),
                                                "rollout_policy_version": int(r.policy_version), "consumed_policy_version": self.policy_version,
                                                "tokens": np.asarray(r.tokens, np.int64), "finish_reason": r.finish_reason}, block=False)
        if self._trajectory_store is None:
            return
        if hasattr(self._trajectory_store, "add_step"):          # a step-level ATIF store
            from ..trajectory import trajectory as T
            from ..trajectory.converter import create_trajectory_metadata, log_trajectory
            for g in groups:
                for i, (p, r) in enumerate(zip(g.payloads, g.responses)):
                    ex = p.example if isinstance(p.example, Mapping) else {}
                    meta = create_trajectory_metadata(f"{r.request_id}", prompt_id=g.prompt_id,
                                                      group_index=int((r.metadata or {}).get("group_index", i)))
                    meta.status, meta.total_reward = "SUCCEEDED", float(p.reward or 0.0)
                    meta.target_policy_versions = [int(p.policy_version)]
                    meta.extra = {"consumed_at_step": step}
                    steps = [T.TunixEnvStep(step_id=0, source="user", message=str(g.item.get("prompt", "")),
                                            env_tokens=np.asarray(ex.get("prompt_ids", ()), np.int64)),
                             T.TunixAgentStep(step_id=1, source="agent", message=r.text or "", llm_call_count=1,
                                              assistant_tokens=np.asarray(r.tokens, np.int64),
                                              assistant_masks=np.ones(len(r.tokens), np.int64),
                                              logprobs=None if r.logprobs is None else np.asarray(r.logprobs, np.float32),
                                              policy_version=int(r.policy_version))]
                    log_trajectory(self._trajectory_store, meta.create_trajectory(steps))
            return
        from ..trajectory.store import new_record
        for g in groups:
            for p in g.payloads:
                ex = p.example if isinstance(p.example, Mapping) else {}
                self._trajectory_store.put(new_record(
                    [{"prompt_ids": np.asarray(ex.get("prompt_ids", ())).tolist(),
                      "completion_ids": np.asarray(ex.get("completion_ids", ())).tolist()}],
                    reward=float(p.reward or 0.0), group_id=g.prompt_id, policy_version=int(p.policy_version), consumed_at_step=step))

    async def train_stage(self) -> None:
        pending: Optional[asyncio.Task] = None
        results: list = []

        async def settle() -> None:
            nonlocal pending
            task, pending = pending, None
            if task is not None:
                results.append(await task)

        async def submit(mb, last: bool) -> None:
            nonlocal pending
            if self.reference_kl:                                # overlaps with the training call that is in flight
                keys = ("input_tokens", "positions", "segment_ids", "prompt_mask", "completion_mask")
                ref = await self.engine.per_token_logps(Role.REFERENCE, {k: mb.arrays[k] for k in keys if k in mb.arrays})
                mb.arrays["ref_per_token_logps"] = np.asarray(ref, np.float32)
            await settle()                                       # one call in flight: the next batch was assembled meanwhile
            pending = asyncio.create_task(self.engine.train_step(mb, role=Role.ACTOR, accumulate_gradients=True,
                                                                 apply_optimizer=last))
        eof = False
        try:
            while not eof and (self.max_steps is None or self._step < self.max_steps):
                step, t0, consumed_version = self._step, time.monotonic(), self.policy_version
                groups, stats, held = [], [], None
                results.clear()
                packing_s = 0.0

                async def take(batches) -> None:
                    nonlocal held
                    for mb in batches:
                        if held is not None:
                            await submit(held, False)
                        held = mb
                        stats.append(mb.stats)
                while len(groups) < self.full_batch_size:
                    g = await self._scored_q.get()
                    if g is _EOF:
                        eof = True
                        break
                    if not groups and self.on_step_begin:
                        self.on_step_begin(step)
                    groups.append(g)
                    if self.mode == "eval":
                        continue
                    tp = time.perf_counter()
                    batches = await asyncio.to_thread(lambda: list(self.assembler.feed(g.payloads)))
                    packing_s += time.perf_counter() - tp
                    await take(batches)
                if not groups:
                    log.info("dataset exhausted at step %d", step)
                    break
                if self.mode == "train":
                    tp = time.perf_counter()
                    batches = await asyncio.to_thread(lambda: list(self.assembler.flush()))
                    packing_s += time.perf_counter() - tp
                    await take(batches)
                    if held is None:
                        raise RuntimeError(f"step {step}: {len(groups)} group(s) produced no micro-batch")
                    await submit(held, True)
                    await settle()
                final = results[-1] if results else None
                payloads = [p for g in groups for p in g.payloads]
                rewards = np.asarray([p.reward or 0.0 for p in payloads], np.float64)
                adv = np.asarray([float(np.mean(p.example["advantages"])) for p in payloads
                                  if isinstance(p.example, Mapping) and p.example.get("advantages") is not None
                                  and np.size(p.example["advantages"])], np.float64)
                if self.mode == "train" and self.checkpoint_every and (step + 1) % self.checkpoint_every == 0:
                    opt_step = final.get("train_step") if isinstance(final, Mapping) else None
                    await self.engine.save_checkpoint(role=Role.ACTOR, metadata={
                        "step": int(opt_step) if opt_step is not None else step + 1, "global_step": step + 1,
                        "policy_version": self.policy_version + (1 if self.sync_weights else 0), "num_rollouts": len(payloads),
                        "num_microbatches": len(stats), **self.dispatch_window.checkpoint_metadata(groups)})
                if self.mode == "train" and self.sync_weights:
                    v = await self.engine.sync_weights(role=Role.ACTOR)
                    self.policy_version = v if v is not None else self.policy_version + 1
                gen_metrics = _generation_metrics([g.responses for g in groups])
                log.info("[pipeline] COMMIT step=%d consumed_version=%d rollout_versions=%s prompts=%s", step, consumed_version,
                         [int(g.responses[0].policy_version) for g in groups], summarize_list([g.prompt_id for g in groups], 8))
                self.dispatch_window.record_committed_groups(groups)
                for g in groups:
                    self._prompts.pop(g.prompt_id, None)
                filtered, self._filtered_groups = self._filtered_groups, []
                losses = [r["loss"] for r in ([x for x in results[:-1]] + ([final.get("fwd_bwd")] if isinstance(final, Mapping) else []))
                          if isinstance(r, Mapping) and r.get("loss") is not None]
                res = RLStepResult(step=step, policy_version=self.policy_version, num_rollouts=len(payloads), num_microbatches=len(stats),
                                   reward_mean=float(rewards.mean()) if rewards.size else 0.0,
                                   reward_std=float(rewards.std()) if rewards.size else 0.0,
                                   advantage_mean=float(adv.mean()) if adv.size else 0.0,
                                   advantage_std=float(adv.std()) if adv.size else 0.0, filtered_groups=len(filtered),
                                   step_time_s=time.monotonic() - t0, train_result=final)
                self.last_step_result = res
                rec = {**dataclasses.asdict(res), "loss": float(np.mean(losses)) if losses else None, "packing_time_s": packing_s,
                       "consumed_policy_version": consumed_version,
                       "staleness_max": max(consumed_version - int(r.policy_version) for g in groups for r in g.responses),
                       **summarize_padding_stats(stats), **gen_metrics}
                rec.pop("train_result")
                self.history.append(rec)
                for name, key in (("rewards/mean", "reward_mean"), ("rewards/std", "reward_std"), ("advantages/mean", "advantage_mean"),
                                  ("actor/loss", "loss"), ("perf/step_time_s", "step_time_s"), ("perf/packing_time_s", "packing_time_s"),
                                  ("batch/padding_ratio", "padding_ratio"), ("rollout/filtered_groups", "filtered_groups"),
                                  ("rollout/staleness_max", "staleness_max")):
                    self._log_metric(name, rec.get(key), step)
                for name, value in gen_metrics.items():
                    self._log_metric(name, value, step)
                self._store_trajectories(groups, step)
                if self.on_step_end:
                    self.on_step_end(step, final)
                self._step += 1
                self.dispatch_window.release()          # after the increment: the dispatcher re-reads the step when it wakes
        finally:
            if pending is not None:
                pending.cancel()
                with contextlib.suppress(asyncio.CancelledError, Exception):
                    await pending

    # ------------------------------------------------------------------ entry points
    async def run_async(self, engine, dataset: Optional[Iterable[Any]] = None, validate: bool = False, **kwargs) -> list:
        self.engine = engine
        if dataset is not None:
            self.dataset = dataset
        if validate:                                    # everything that is wrong with the set-up, in one error
            from .startup_validation import validate_program
            validate_program(self, engine)
        self._dispatch_done = asyncio.Event()
        self._raw_q: asyncio.Queue = asyncio.Queue()
        self._scored_q: asyncio.Queue = asyncio.Queue()
        self._in_flight = self._dispatched = 0
        self._order_next, self._order_pending = 0, {}
        # before any stage starts: the train loop's bound and the dataset prefix to skip both come from the restored step
        if self.mode == "train":
            await self._resume_from_checkpoint()
        self._base_step = self._step
        if self.mode == "train":
            engine.configure_worker(role=Role.ACTOR, algo=self.algo, assembler=self.assembler)
        if self.mode == "train" and self.sync_weights and self._step == 0:           # a resumed run has just pushed the restored weights
            await engine.prepare_rollout_policy(role=Role.ACTOR, sync_weights=True, policy_version=self.policy_version)
        train = asyncio.create_task(self.train_stage())
        tasks = [asyncio.create_task(self.rollout_dispatch_stage()), asyncio.create_task(self.polling_stage()),
                 asyncio.create_task(self.critique_stage()), train]
        waiting = set(tasks)
        try:
            while not train.done() and waiting:
                done, waiting = await asyncio.wait(waiting, return_when=asyncio.FIRST_COMPLETED, timeout=0.05)
                for t in done:
                    if t.exception() is not None:
                        raise t.exception()
            if train.exception() is not None:
                raise train.exception()
        except BaseException:
            for t in tasks:
                t.cancel()
            with contextlib.suppress(asyncio.CancelledError, Exception):
                await asyncio.gather(*tasks, return_exceptions=True)
            self.assembler.reset()
            raise
        finally:
            for t in tasks:
                if not t.done():
                    t.cancel()
            with contextlib.suppress(asyncio.CancelledError, Exception):
                await asyncio.gather(*tasks, return_exceptions=True)
        return self.history

    def run(self, engine, dataset: Optional[Iterable[Any]] = None, **kwargs):
        """Blocking entry point; from inside a running event loop it schedules the run and returns the task."""
        try:
            loop = asyncio.get_running_loop()
        except RuntimeError:
            loop = None
        if loop is not None and loop.is_running():
            self._bg_task = loop.create_task(self.run_async(engine, dataset, **kwargs))     # kwargs: validate=...
            self._bg_task.add_done_callback(lambda t: t.cancelled() or t.exception())
            return self._bg_task
        return asyncio.run(self.run_async(engine, dataset, **kwargs))
