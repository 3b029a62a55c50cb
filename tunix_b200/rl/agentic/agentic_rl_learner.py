"""Agentic (multi-turn, asynchronous) RL learner (tunix/rl/agentic/agentic_rl_learner.py:105-1303).

A dedicated asyncio loop thread runs the producer: prompts -> (agent, env) pairs x G -> `RolloutOrchestrator`
(bounded concurrency) -> complete groups -> `TrainExample`s -> a thread-safe queue. The main thread consumes
groups as they arrive and trains; after every prompt batch it takes the weight-sync side of a
`RolloutSyncLock` (waits for in-flight model calls, blocks new ones), syncs weights, bumps `policy_version`
and lets the producer continue. `off_policy_steps` bounds how many prompt batches the producer may run
ahead of the trainer (:838-847). Model calls from concurrent episodes are gathered by a micro-batcher so the
rollout engine sees batches, not single prompts (the reference relies on vLLM server mode for this, :293-301).
"""
from __future__ import annotations

import abc
import asyncio
import concurrent.futures as cf
import queue
import threading
import time
from typing import Any, Callable, Iterable, Optional, Sequence

import logging

import numpy as np
import torch

from ...common.datatypes import Mode
from .. import algo_core, common, function_registry, reward_manager as _reward_manager  # noqa: F401 (registrations)
from ..rl_cluster import RLCluster
from .agents.model_agent import ModelAgent
from .environments.task_environment import TaskEnvironment
from .pipeline.rollout_orchestrator import RolloutOrchestrator
from .trajectory.trajectory_collect_engine import TrajectoryCollectEngine
from .utils import RolloutSyncLock


log = logging.getLogger(__name__)


class _ModelCallBatcher:
    """Collects concurrent single-prompt model calls for a short window and serves them with one engine call."""

    def __init__(self, generate_fn: Callable[[list, Optional[int]], list], max_batch: int = 64, window_s: float = 0.002):
        self._gen, self._max, self._win = generate_fn, max_batch, window_s
        self._pending: list = []
        self._lock = asyncio.Lock()
        self._flusher: Optional[asyncio.Task] = None
        self._pool = cf.ThreadPoolExecutor(max_workers=1, thread_name_prefix="agentic-gen")

    async def call(self, prompt_token_ids: list, max_tokens: Optional[int]) -> dict:
        fut = asyncio.get_running_loop().create_future()
        async with self._lock:
            self._pending.append((prompt_token_ids, max_tokens, fut))
            if self._flusher is None or self._flusher.done():
                self._flusher = asyncio.create_task(self._flush_later())
        return await fut

    async def _flush_later(self):
        await asyncio.sleep(self._win)
        while True:
            async with self._lock:
                batch, self._pending = self._pending[: self._max], self._pending[self._max:]
            if not batch:
                return
            prompts = [b[0] for b in batch]
            budget = min((b[1] for b in batch if b[1] is not None), default=None)
            try:
                outs = await asyncio.get_running_loop().run_in_executor(self._pool, self._gen, prompts, budget)
                for (_, _, fut), o in zip(batch, outs):
                    if not fut.done():
                        fut.set_result(o)
            except Exception as e:
                for _, _, fut in batch:
                    if not fut.done():
                        fut.set_exception(e)

    def close(self):
        self._pool.shutdown(wait=False, cancel_futures=True)


class AgenticRLLearner(abc.ABC):
    def __init__(self, rl_cluster: RLCluster, reward_fns, algo_config, *, agent_class=ModelAgent, agent_kwargs=None,
                 env_class=TaskEnvironment, env_kwargs=None, chat_parser=None, max_concurrency: int = 16,
                 off_policy_steps: int = 0, max_turns: int = 1, episode_timeout: float = 600.0, metric_fns=None,
                 server_mode: bool = False, model_client=None, pack_first: bool = False, pack_budget: Optional[int] = None,
                 trajectory_logger=None):
        """`model_client`: an `async (chat_completions, prompt_token_ids, max_tokens) -> {"text", "tokens",
        "logprobs"}` that replaces the cluster's own rollout engine for the episodes' model calls, e.g.
        `http_model_client.HTTPModelClient` in front of engines in another process. Keeping those engines' weights
        current is then the deployment's job (`experimental.weight_sync`)."""
        self.model_client = model_client
        # pack first (tunix/rl/agentic/agentic_grpo_learner.py:338-442,649): the groups of a prompt batch are packed
        # into rows of `pack_budget` tokens BEFORE the reference (and, when asked for, the old-policy) log-probs are
        # computed, so that those forward passes run on dense packed rows instead of rows padded to the longest
        # conversation of a group
        self.pack_first, self.pack_budget = pack_first, pack_budget
        self.trajectory_logger = trajectory_logger      # object with .log(items) or a callable; gets every finished group
        self.rl_cluster, self.algo_config = rl_cluster, algo_config
        self.tcfg = rl_cluster.cluster_config.training_config
        self.agent_class, self.agent_kwargs = agent_class, dict(agent_kwargs or {})
        self.env_class, self.env_kwargs = env_class, dict(env_kwargs or {})
        self.chat_parser = chat_parser
        self.max_concurrency, self.off_policy_steps = max_concurrency, off_policy_steps
        # server mode: every model call is submitted on its own to the paged engine's server and joins the running
        # batch there; otherwise concurrent calls are collected for a short window into one engine call
        self.server_mode = server_mode
        self._server = None
        self._server_pool = None
        self.max_turns, self.episode_timeout = max_turns, episode_timeout
        self.metric_fns = list(metric_fns or [])
        self.reward_manager = None
        if reward_fns:
            cls = function_registry.get_reward_manager("agentic-sequence-level")
            self.reward_manager = cls(reward_fns, algo_config)
        self.policy_version = int(rl_cluster.global_steps)      # a resumed run goes on counting from the restored step
        self.stale_dropped = 0
        self.sync_lock = RolloutSyncLock()
        self.pad_id, self.eos_id = rl_cluster.rollout.pad_id(), rl_cluster.rollout.eos_id()
        self.device = next(rl_cluster.train_actor.parameters()).device
        rc = rl_cluster._rollout_config(Mode.TRAIN)
        self.algo_config.temperature = rc.temperature if rc.temperature and rc.temperature > 0 else None
        self._loop = asyncio.new_event_loop()
        self._thread = threading.Thread(target=self._loop.run_forever, name="agentic-loop", daemon=True)
        self._thread.start()
        self._batcher: Optional[_ModelCallBatcher] = None

    # ---------------------------------------------------------------- model
    def _generate_batch(self, prompts: list, max_tokens: Optional[int]) -> list:
        import dataclasses
        rc = self.rl_cluster._rollout_config(Mode.TRAIN)
        if max_tokens is not None:
            rc = dataclasses.replace(rc, max_tokens_to_generate=min(rc.max_tokens_to_generate, max_tokens))
        with self.sync_lock.acquire_rollout():
            out = self.rl_cluster.rollout.generate(None, rc, prompt_token_ids=prompts)
        res = []
        for i in range(len(prompts)):
            lp = out.logprobs[i] if out.logprobs is not None else np.zeros(len(out.tokens[i]), np.float32)
            res.append({"text": out.text[i], "tokens": np.asarray(out.tokens[i]), "logprobs": np.asarray(lp, np.float32),
                        "policy_version": self.policy_version})
        return res

    def _server_call(self, prompt_token_ids, max_tokens) -> dict:
        with self.sync_lock.acquire_rollout():
            toks, lps = self._server.generate(prompt_token_ids, max_tokens)
            version = self.policy_version
        tk = self.rl_cluster.tokenizer
        stop = {tk.eos_id(), tk.pad_id()}
        return {"text": tk.decode([int(t) for t in toks if int(t) not in stop]), "tokens": toks, "logprobs": lps,
                "policy_version": version}

    async def _model_call(self, chat_completions=None, prompt_token_ids=None, max_tokens=None) -> dict:
        if self.model_client is not None:
            return await self.model_client(chat_completions=chat_completions, prompt_token_ids=prompt_token_ids, max_tokens=max_tokens)
        if self._server is not None:
            return await asyncio.get_running_loop().run_in_executor(self._server_pool, self._server_call,
                                                                   list(prompt_token_ids), max_tokens)
        return await self._batcher.call(prompt_token_ids, max_tokens)

    # ------------------------------------------------------------- producer
    def _make_pairs(self, batch: dict, batch_idx: int):
        G = self.algo_config.num_generations
        tasks = batch.get("tasks")
        if tasks is None:
            prompts = batch["prompts"]
            answers = batch.get("answer", [None] * len(prompts))
            tasks = [{"question": p, "answer": a} for p, a in zip(prompts, answers)]
        for pi, task in enumerate(tasks):
            for _ in range(G):
                yield self.agent_class(**self.agent_kwargs), self.env_class(task=task, **self.env_kwargs), (batch_idx, pi)

    def _engine_factory(self, agent, env):
        rc = self.rl_cluster._rollout_config(Mode.TRAIN)
        return TrajectoryCollectEngine(agent, env, model_call=self._model_call, tokenizer=self.rl_cluster.tokenizer,
                                       chat_parser=self.chat_parser, max_steps=self.max_turns, timeout=self.episode_timeout,
                                       max_response_length=rc.max_tokens_to_generate)

    async def _produce(self, batches: Iterable[dict], out_q: queue.Queue, permits: threading.Semaphore):
        self._batcher = _ModelCallBatcher(self._generate_batch, max_batch=self.max_concurrency)
        start = getattr(self.rl_cluster.rollout, "start_server", None) if self.server_mode else None
        if start is not None:
            self._server = start(self.rl_cluster._rollout_config(Mode.TRAIN))
            if self._server is not None:
                self._server_pool = cf.ThreadPoolExecutor(max_workers=self.max_concurrency, thread_name_prefix="agentic-call")
        try:
            for bi, batch in enumerate(batches):
                await asyncio.get_running_loop().run_in_executor(None, permits.acquire)
                orch = RolloutOrchestrator(engine_factory=self._engine_factory, group_size=self.algo_config.num_generations,
                                           max_concurrency=self.max_concurrency)
                prod = asyncio.create_task(orch.run_producers_from_stream(self._make_pairs(batch, bi)))
                async for groups in orch.yield_batches(1):
                    for g in groups:
                        out_q.put(("group", bi, g))
                await prod
                out_q.put(("batch_end", bi, None))
        except BaseException as e:
            out_q.put(("error", -1, e))
        finally:
            self._batcher.close()
            if self._server is not None:
                self._server_pool.shutdown(wait=False, cancel_futures=True)
                self._server.close()
                self._server = None
            out_q.put(("done", -1, None))

    # ------------------------------------------------------------- consumer
    @abc.abstractmethod
    def _process_group(self, items: list, defer_logps: bool = False) -> Optional[common.TrainExample]: ...

    def _log_trajectories(self, items: list) -> None:
        lg = self.trajectory_logger
        if lg is None:
            return
        rows = [{"episode_id": getattr(it, "episode_id", None), "group_id": getattr(it, "group_id", None),
                 "policy_version": self.policy_version, **{k: (v.tolist() if hasattr(v, "tolist") else v)
                                                           for k, v in getattr(it, "traj", {}).items()}} for it in items]
        (lg.log if hasattr(lg, "log") else lg)(rows)

    def _pack_and_score(self, examples: list) -> list:
        """Pack the step's examples into dense rows, then compute the deferred log-probs on the packed rows."""
        from .. import utils as rl_utils
        rc = self.rl_cluster._rollout_config(Mode.TRAIN)
        budget = self.pack_budget or self.tcfg.max_seq_token_per_tpu or (rc.max_prompt_length + rc.max_tokens_to_generate)
        longest = max(int(e.prompt_mask.sum(1).max()) + int((e.completion_ids != self.pad_id).sum(1).max()) for e in examples)
        budget = max(budget, longest)
        packed = list(rl_utils.pack_sequences(examples, budget, pack_size=max(self.tcfg.train_micro_batch_size or 1, 1),
                                              pad_id=self.pad_id, device=self.device,
                                              max_segments=self.tcfg.max_segments_per_packed_row))
        beta = getattr(self.algo_config, "beta", 0.0)
        for ex in packed:
            if beta != 0.0:
                ex.ref_per_token_logps = self.rl_cluster.get_ref_per_token_logps(
                    ex.prompt_ids, ex.completion_ids, self.pad_id, self.eos_id, completion_mask=ex.completion_mask,
                    temperature=self.algo_config.temperature, segment_ids=ex.segment_ids,
                    segment_positions=ex.segment_positions)
            if not self.algo_config.use_rollout_logps and ex.old_per_token_logps is None:
                # no update has happened since the last weight sync: the actor's weights are the sampler's
                ex.old_per_token_logps = self.rl_cluster.get_actor_per_token_logps(
                    ex.prompt_ids, ex.completion_ids, self.pad_id, self.eos_id, completion_mask=ex.completion_mask,
                    temperature=self.algo_config.temperature, segment_ids=ex.segment_ids,
                    segment_positions=ex.segment_positions)
        return packed

    def evaluate(self, eval_ds: Iterable[dict]) -> dict:
        """Run the agentic loop over `eval_ds` without training: mean trajectory reward, share of valid episodes and
        turns per episode, logged in eval mode (the reference evaluates inside its agentic loop every
        `eval_every_n_steps`)."""
        async def run():
            self._batcher = self._batcher or _ModelCallBatcher(self._generate_batch, max_batch=self.max_concurrency)
            rewards, valid, turns = [], [], []
            for bi, batch in enumerate(eval_ds):
                orch = RolloutOrchestrator(engine_factory=self._engine_factory, group_size=self.algo_config.num_generations,
                                           max_concurrency=self.max_concurrency)
                prod = asyncio.create_task(orch.run_producers_from_stream(self._make_pairs(batch, bi)))
                async for groups in orch.yield_batches(1):
                    for g in groups:
                        for it in g:
                            rewards.append(float(it.traj["trajectory_reward"]))
                            valid.append(it.traj["status"] not in _INVALID)
                            turns.append(it.traj["num_turns"])
                await prod
            return rewards, valid, turns
        from .agents.agent_types import INVALID_TRAJECTORY_STATUSES as _INVALID
        rewards, valid, turns = asyncio.run_coroutine_threadsafe(run(), self._loop).result()
        out = {"eval/rewards/mean": float(np.mean(rewards)) if rewards else 0.0,
               "eval/trajectory/valid_frac": float(np.mean(valid)) if valid else 0.0,
               "eval/trajectory/num_turns": float(np.mean(turns)) if turns else 0.0, "eval/episodes": len(rewards)}
        self.rl_cluster.buffer_metrics({k: (v, np.mean) for k, v in out.items()}, Mode.EVAL)
        self.rl_cluster.flush_metrics()
        return out

    def train(self, train_ds: Iterable[dict], eval_ds=None) -> None:
        out_q: queue.Queue = queue.Queue()
        permits = threading.Semaphore(self.off_policy_steps + 1)
        max_steps = self.tcfg.max_steps
        it = iter(train_ds)
        for _ in range(self.rl_cluster.global_steps):   # resume: skip consumed prompt batches
            next(it, None)
        fut = asyncio.run_coroutine_threadsafe(self._produce(it, out_q, permits), self._loop)
        mu = getattr(self.algo_config, "num_iterations", 1)
        pending: list = []
        try:
            while True:
                kind, bi, payload = out_q.get()
                if kind == "error":
                    raise RuntimeError("agentic rollout producer failed") from payload
                if kind == "done":
                    break
                if kind == "group":
                    self._log_trajectories(payload)
                    ex = self._process_group(payload, defer_logps=self.pack_first)
                    if ex is not None and self._too_old(ex):
                        ex = None
                    if ex is not None:
                        pending.append(ex)
                        if not self.pack_first:
                            self.rl_cluster.update_actor([ex], None)
                    continue
                # batch_end: (pack-first: pack, score and train now;) extra iterations over the collected groups,
                # then weight sync under the lock
                if self.pack_first and pending:
                    pending = self._pack_and_score(pending)
                    self.rl_cluster.update_actor(list(pending), None)
                for _ in range(1, mu):
                    self.rl_cluster.update_actor(list(pending), None)
                pending = []
                with self.sync_lock.acquire_weight_sync():
                    srv = self._server
                    if srv is not None:
                        srv.pause()             # no request is in flight under the lock; the server parks its loop
                    self.rl_cluster.sync_weights()
                    self.policy_version += 1
                    if srv is not None:
                        srv.resume()            # re-reads the updated weights before the next admission
                self.rl_cluster.flush_metrics()
                if eval_ds is not None and self.tcfg.eval_every_n_steps and \
                        self.rl_cluster.global_steps % self.tcfg.eval_every_n_steps == 0:
                    self.evaluate(eval_ds)
                permits.release()
                if max_steps is not None and self.rl_cluster.global_steps >= max_steps:
                    break
        finally:
            fut.cancel()
            for _ in range(self.off_policy_steps + 2):      # a producer parked on the permit must not outlive the loop
                permits.release()
            self.close()

    def _too_old(self, ex) -> bool:
        """A group generated more than `off_policy_steps` weight versions ago is not trained on
        (tunix/rl/agentic/agentic_rl_learner.py:1273-1303); a version of -1 or None means "unknown" and passes."""
        v = getattr(ex, "policy_version", None)
        if v is None or int(v) < 0 or self.policy_version - int(v) <= self.off_policy_steps:
            return False
        self.stale_dropped += 1
        log.warning("skipping a group generated at policy version %d: current version %d, off_policy_steps %d", int(v),
                    self.policy_version, self.off_policy_steps)
        self.rl_cluster.buffer_metrics({"trajectory/stale_dropped": (1.0, np.sum)}, Mode.TRAIN)
        return True

    def close(self) -> None:
        self.rl_cluster.close()
        if self.reward_manager is not None and hasattr(self.reward_manager, "close"):
            self.reward_manager.close()
        self._loop.call_soon_threadsafe(self._loop.stop)
