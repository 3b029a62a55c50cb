"""Concurrency core of a rollout worker (tunix/experimental/rollout/manager.py:38-480).

`RolloutManager` runs episodes as asyncio tasks against one generation engine, streams them back in completion
order, and runs the three barriers of a weight-sync round on top of the `TrafficController`:

  pre_weight_sync   close admission; wait for the episodes in flight (or, with `partial_rollout`, let them
                    continue after the sync with the new policy: each call they make notes the version it used)
  weight_sync       install the weights through `apply_weights(version, payload)`
  post_weight_sync  set the policy version, reopen admission
  abort_weight_sync reopen without a version change

An episode is `episode_fn(model_call, item) -> result`, where `model_call(prompt_token_ids, max_tokens)` is a
coroutine that goes to the engine: an `EngineServer` (requests join its running batch) or a blocking
`generate(prompt_token_ids, max_tokens) -> (tokens, logprobs)` callable, which is run on a thread."""
from __future__ import annotations

import asyncio
import time
from typing import Any, AsyncIterator, Awaitable, Callable, Optional

from ..worker.traffic_controller import AdmissionClosedError, TrafficController


class RolloutManager:
    def __init__(self, engine, episode_fn: Callable[..., Awaitable[Any]], *, max_concurrency: int = 64,
                 apply_weights: Optional[Callable[[int, Any], None]] = None, partial_rollout: bool = False,
                 drain_timeout_s: float = 300.0):
        self.engine, self.episode_fn = engine, episode_fn
        self._apply = apply_weights
        self.partial_rollout, self.drain_timeout_s = partial_rollout, drain_timeout_s
        self.traffic = TrafficController()
        self._slots = asyncio.Semaphore(max_concurrency)
        self._done: asyncio.Queue = asyncio.Queue()
        self.policy_version = 0
        self.stats = {"episodes": 0, "model_calls": 0, "failed": 0}

    # ------------------------------------------------------------------ serving
    async def model_call(self, prompt_token_ids, max_tokens: Optional[int] = None) -> dict:
        """One generation request of an episode. With partial rollouts a request made while a sync is in progress
        waits at the gate, so no request straddles a weight update; without them the episodes in flight are being
        drained and their requests pass."""
        if self.partial_rollout:
            await self.traffic.wait_for_admission()
        self.stats["model_calls"] += 1
        version = self.policy_version
        if hasattr(self.engine, "submit"):
            toks, lps = await asyncio.wrap_future(self.engine.submit(list(prompt_token_ids), max_tokens))
        else:
            toks, lps = await asyncio.get_running_loop().run_in_executor(None, self.engine, list(prompt_token_ids), max_tokens)
        return {"tokens": toks, "logprobs": lps, "policy_version": version}

    async def _run(self, item) -> None:
        async with self._slots:
            t0 = time.monotonic()
            try:
                res = await self.episode_fn(self.model_call, item)
                self.stats["episodes"] += 1
                await self._done.put({"item": item, "result": res, "error": None, "seconds": time.monotonic() - t0})
            except asyncio.CancelledError:
                await self._done.put({"item": item, "result": None, "error": asyncio.CancelledError(), "seconds": 0.0})
                raise
            except Exception as e:                      # an episode's failure is data, not the manager's failure
                self.stats["failed"] += 1
                await self._done.put({"item": item, "result": None, "error": e, "seconds": time.monotonic() - t0})

    def start_episode(self, item) -> "asyncio.Task":
        task = asyncio.ensure_future(self._run(item))
        if not self.traffic.try_admit(task):
            raise AdmissionClosedError(f"admission is closed ({self.traffic.state.value})")
        return task

    async def pop_next_completed(self) -> dict:
        return await self._done.get()

    async def as_completed(self, items) -> AsyncIterator[dict]:
        """Start an episode per item (waiting at the gate while a sync is in progress) and yield the outcomes in
        completion order."""
        n = 0
        for it in items:
            await self.traffic.wait_for_admission()
            self.start_episode(it)
            n += 1
        for _ in range(n):
            yield await self._done.get()

    # --------------------------------------------------------------- weight sync
    async def pre_weight_sync(self) -> dict:
        t0 = time.monotonic()
        before = len(self.traffic.active_tasks())
        self.traffic.close_for_sync()
        drained = True
        if not self.partial_rollout:
            drained = await self.traffic.drain(self.drain_timeout_s)
        if hasattr(self.engine, "pause"):
            await asyncio.get_running_loop().run_in_executor(None, self.engine.pause, self.drain_timeout_s)
        return {"in_flight_before": before, "in_flight_after": len(self.traffic.active_tasks()), "drained": drained,
                "seconds": time.monotonic() - t0}

    async def weight_sync(self, version: int, payload: Any = None) -> int:
        if self._apply is not None:
            await asyncio.get_running_loop().run_in_executor(None, self._apply, version, payload)
        self._pending_version = int(version)
        return int(version)

    async def post_weight_sync(self) -> bool:
        self.policy_version = getattr(self, "_pending_version", self.policy_version)
        if hasattr(self.engine, "resume"):
            self.engine.resume()
        return self.traffic.reopen()

    async def abort_weight_sync(self) -> bool:
        if hasattr(self.engine, "resume"):
            self.engine.resume()
        return self.traffic.reopen()

    def cancel_all(self) -> list:
        return self.traffic.stop()
