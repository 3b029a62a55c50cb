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
                 server_mode: bool = False, model_client=None):
        """`model_client`: an `async (chat_completions, prompt_token_ids, max_tokens) -> {"text", "tokens",
        "logprobs"}` that replaces the cluster's own rollout engine for the episodes' model calls, e.g.
        `http_model_client.HTTPModelClient` in front of engines in another process. Keeping those engines' weights
        current is then the deployment's job (`experimental.weight_sync`)."""
        self.model_client = model_client
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
        self.policy_version = 0
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
    def _process_group(self, items: list) -> Optional[common.TrainExample]: ...

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
                    ex = self._process_group(payload)
                    if ex is not None:
                        pending.append(ex)
                        self.rl_cluster.update_actor([ex], None)
                    continue
                # batch_end: extra iterations over the collected groups, then weight sync under the lock
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
                permits.release()
                if max_steps is not None and self.rl_cluster.global_steps >= max_steps:
                    break
        finally:
            fut.cancel()
            self.close()

    def close(self) -> None:
        self.rl_cluster.close()
        if self.reward_manager is not None and hasattr(self.reward_manager, "close"):
            self.reward_manager.close()
        self._loop.call_soon_threadsafe(self._loop.stop)
