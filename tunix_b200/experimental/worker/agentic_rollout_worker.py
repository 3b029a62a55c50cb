"""A rollout worker that runs whole episodes: agent + environment + sampler
(tunix/experimental/worker/rollout_worker.py, the multi-turn path over experimental/rollout/collector.py).

A `RolloutRequest` names its agent and environment (`metadata["agent"]`, `metadata["env"]`: keys of the agent /
environment registries, or classes; kwargs under `agent_kwargs` / `env_kwargs`; the task under `task` or
`env_config`). The worker builds them, runs the episode through a `TrajectoryCollectorEngine` against its asynchronous
sampler on a private event loop, and answers with a `RolloutResponse` whose tokens are the whole conversation after the
prompt, whose metadata carries what training needs beyond tokens and log-probs: `conversation_masks` (1 = the model's
tokens), `prompt_token_ids`, `trajectory_reward` (the environment's), `status`, `num_turns`, `policy_versions`, and the
collector's `raw_length` / `clipped` facts.

Weight sync: running episodes are paused before their next model call, the sampler's three-phase sync runs, the
episodes go on under the new weights (each turn notes its version). `stop()` cancels what is still running."""
from __future__ import annotations

import asyncio
import dataclasses
import threading
from typing import Any, Callable, Collection, Optional

import numpy as np

from ...rl.agentic.agents import agent_types
from ..common.datatypes import RolloutRequest, RolloutResponse
from ..orchestrator.worker_registry import WorkerInfo
from ..rl.agentic import registry as registries
from ..rollout.collector import TrajectoryCollectorEngine
from .abstract_worker import AbstractWorker


@dataclasses.dataclass
class _EpisodeRequest:
    """What the collector reads off a request."""
    prompt_id: str
    group_index: int
    generation_kwargs: dict
    max_turns: int
    max_response_length: Optional[int]
    target_policy_version: int
    metadata: dict


def _resolve(kind: str, spec, registry: registries.Registry):
    if isinstance(spec, type):
        return spec
    if spec is None:
        raise ValueError(f"the request names no {kind} (metadata[{kind!r}])")
    return registry.get(str(spec))


class AgenticRolloutWorker(AbstractWorker):
    role = "rollout"

    def __init__(self, worker_id: str, sampler, tokenizer, *, chat_parser=None, eos_ids: Optional[Collection[int]] = None,
                 default_agent=None, default_env=None, apply_weights: Optional[Callable[[int, Any], None]] = None,
                 max_inflight: int = 64, needs_seed: bool = True, on_report=None):
        super().__init__(worker_id, max_inflight=max_inflight, on_report=on_report)
        self.sampler, self.tokenizer, self.chat_parser = sampler, tokenizer, chat_parser
        self.eos_ids = list(eos_ids or [])
        self.default_agent, self.default_env = default_agent, default_env
        self._apply, self.needs_seed = apply_weights, needs_seed
        self._loop: Optional[asyncio.AbstractEventLoop] = None
        self._thread: Optional[threading.Thread] = None
        self._episodes: set = set()
        self._ep_lock = threading.Lock()
        self.served = 0

    def info(self) -> WorkerInfo:
        return WorkerInfo(self.worker_id, (self.role,), attributes={"episodes": True})

    # ------------------------------------------------------------------ lifecycle
    def _initialize(self) -> bool:
        self._loop = asyncio.new_event_loop()
        self._thread = threading.Thread(target=self._loop.run_forever, name=f"{self.worker_id}-episodes", daemon=True)
        self._thread.start()
        if hasattr(self.sampler, "initialize"):
            self.sampler.initialize()
        if hasattr(self.sampler, "start"):
            asyncio.run_coroutine_threadsafe(self.sampler.start(), self._loop).result(60)
        return False

    def _drain(self) -> None:
        with self._ep_lock:
            running = list(self._episodes)
        for ep in running:
            ep.cancel()
        if self._loop is not None:
            if hasattr(self.sampler, "stop"):
                try:
                    asyncio.run_coroutine_threadsafe(self.sampler.stop(), self._loop).result(30)
                except Exception:
                    pass
            self._loop.call_soon_threadsafe(self._loop.stop)
            self._thread.join(5)

    # ------------------------------------------------------------------ one episode
    def _build(self, req: RolloutRequest):
        md = dict(req.metadata or {})
        agent_cls = _resolve("agent", md.get("agent", self.default_agent), registries.AGENT_REGISTRY)
        env_cls = _resolve("env", md.get("env", self.default_env), registries.ENV_REGISTRY)
        task = md.get("task", md.get("env_config"))
        agent = agent_cls(**dict(md.get("agent_kwargs") or {}))
        env = env_cls(task, **dict(md.get("env_kwargs") or {}))
        gen = {"temperature": req.temperature, "top_p": req.top_p, "top_k": req.top_k, "seed": req.seed, "max_tokens": req.max_tokens}
        ereq = _EpisodeRequest(prompt_id=str(req.group_id or md.get("prompt_id", req.request_id)), group_index=int(md.get("group_index", 0)),
                               generation_kwargs={k: v for k, v in gen.items() if v is not None},
                               max_turns=int(md.get("max_turns", 10)), max_response_length=md.get("max_response_length"),
                               target_policy_version=max(int(req.policy_version), int(self.policy_version)),
                               metadata={k: md[k] for k in ("episode_timeout", "overlong_filter") if k in md})
        return TrajectoryCollectorEngine(req.request_id, ereq, self.sampler, env, agent, self.tokenizer, chat_parser=self.chat_parser,
                                         eos_ids=self.eos_ids, policy_version_fn=lambda: self.policy_version, needs_seed=self.needs_seed)

    def _handle(self, req: RolloutRequest) -> RolloutResponse:
        ep = self._build(req)
        with self._ep_lock:
            self._episodes.add(ep)
        try:
            item = asyncio.run_coroutine_threadsafe(ep.run_episode(), self._loop).result()
        finally:
            with self._ep_lock:
                self._episodes.discard(ep)
        self.served += 1
        traj = item.traj
        toks = np.asarray(traj["conversation_tokens"]).astype(np.int64)
        status = traj.get("status")
        invalid = status in agent_types.INVALID_TRAJECTORY_STATUSES or len(toks) == 0
        meta = {**dict(req.metadata or {}), **{k: v for k, v in item.metadata.items() if k in ("raw_length", "clipped", "policy_versions")},
                "conversation_masks": [int(x) for x in np.asarray(traj["conversation_masks"])],
                "prompt_token_ids": [int(x) for x in np.asarray(traj["prompt_tokens"])],
                "trajectory_reward": float(traj.get("trajectory_reward", 0.0)), "status": getattr(status, "name", str(status)),
                "num_turns": int(traj.get("num_turns", 0)), "masked_out": bool(traj.get("masked_out", False)),
                "is_valid": not invalid}
        if traj.get("episode_summary") is not None:
            meta["episode_summary"] = traj["episode_summary"]
        versions = item.metadata.get("policy_versions") or [self.policy_version]
        return RolloutResponse(req.request_id, [int(t) for t in toks], [float(x) for x in np.asarray(traj["old_logprobs"])], None,
                               policy_version=int(min(versions)), finish_reason="stop" if not invalid else "error",
                               group_id=req.group_id, metadata=meta)

    # ------------------------------------------------------------------ weights
    def sync_weights(self, version: int, payload: Any = None) -> None:
        """Unlike a single-call worker this one takes new weights while episodes are in flight: they are paused around
        the swap and stay admitted, so the worker remains BUSY instead of passing through SYNCING."""
        from ..common.datatypes import WorkerState
        if self.state != WorkerState.BUSY:
            return super().sync_weights(version, payload)
        try:
            self._sync_weights(version, payload)
            self.policy_version = version
            self.report(f"synced to version {version} with episodes in flight")
        except BaseException as e:
            self._fail(e)
            raise

    def _sync_weights(self, version: int, payload: Any) -> None:
        with self._ep_lock:
            running = list(self._episodes)
        for ep in running:
            ep.pause()                                   # takes effect before the episode's next model call
        run = lambda coro: asyncio.run_coroutine_threadsafe(coro, self._loop).result(600)     # noqa: E731
        staged = False
        try:
            if hasattr(self.sampler, "pre_weight_sync"):
                run(self.sampler.pre_weight_sync(version))
                staged = True
            if self._apply is not None:
                self._apply(version, payload)
            if hasattr(self.sampler, "weight_sync"):
                run(self.sampler.weight_sync(version))
            if hasattr(self.sampler, "post_weight_sync"):
                run(self.sampler.post_weight_sync(version))
            staged = False
        finally:
            if staged and hasattr(self.sampler, "abort_weight_sync"):
                try:
                    run(self.sampler.abort_weight_sync())
                except Exception:
                    pass
            for ep in running:
                ep.resume()
