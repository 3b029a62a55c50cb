"""`AbstractRLEngine` over this package's workers (tunix/experimental/orchestrator/distributed_rl_engine.py:75-771).

Workers are `AbstractWorker`s in this process or `RemoteWorker` proxies of workers served elsewhere: both answer
`submit(request)` (blocking) and `sync_weights(version, payload)`. The engine turns those blocking calls into
coroutines on a private thread pool so that a program's stages overlap:

* rollouts: prompts become `RolloutRequest`s (`req_<prompt id>_g<index>_v<version>`, the prompt id is the group id
  and the routing key, so the G generations of a prompt share a worker's prefix cache; a deterministic seed per
  (prompt id, index) unless the dispatch gives one); `RoutingPool` picks the worker and retries a failed request on
  the next choice for its key. Dispatch returns at once; finished responses wait in a queue for `poll_rollouts`.
  A request that failed on every worker is reported as a response with `finish_reason="error"` and
  `metadata["is_valid"] = False`, so a program's in-flight count always reaches zero;
* scoring / log-probs go to the inference worker of the role (`{"op": ..., **arrays}`), or to the trainer worker's
  `fwd_only` when no inference worker serves the role;
* `train_step` is `fwd_bwd` (+ `update` with `apply_optimizer`) on the role's trainer worker;
* `sync_weights` runs a round of a `WeightSyncCoordinator` (anything with `run_round(version)`), or, without one,
  hands `export_weights()` to every live rollout worker's `sync_weights`;
* `resume_from_checkpoint` restores the trainer, reads the checkpoint's metadata and realigns the policy version:
  the recorded `policy_version` when the checkpoint carries off-policy state (committed / skipped prompt ids),
  otherwise the restored step boundary.
"""
from __future__ import annotations

import asyncio
import concurrent.futures as cf
import logging
import queue
import time
from typing import Any, Callable, Mapping, Optional, Sequence

from ..common.datatypes import GenerationArgs, Role, RolloutRequest, RolloutResponse, role_name
from ..common.lineage import LineageContext
from ..rollout.collector import generate_vanilla_rollout_seed
from ..weight_sync.weight_sync_coordinator import RoundState
from ..worker.routing import RoutingPool

log = logging.getLogger(__name__)
_REQUEST_FIELDS = ("max_tokens", "temperature", "top_p", "top_k", "seed")


def _get(item, key, default=None):
    return item.get(key, default) if isinstance(item, Mapping) else getattr(item, key, default)


def _named(workers) -> dict:
    if isinstance(workers, Mapping):
        return {str(k): w for k, w in workers.items()}
    return {str(getattr(w, "worker_id", i)): w for i, w in enumerate(workers or ())}


def _by_role(workers) -> dict:
    return {role_name(r): w for r, w in (workers or {}).items()}


class _Routed:
    """A request with the key `RoutingPool` places it by."""
    __slots__ = ("request", "route_key")

    def __init__(self, request: RolloutRequest):
        self.request, self.route_key = request, request.group_id


class DistributedRLEngine:
    def __init__(self, rollout_workers, trainer_workers: Mapping[Any, Any], inference_workers: Optional[Mapping[Any, Any]] = None, *,
                 weight_sync: Any = None, export_weights: Optional[Callable[[], Any]] = None, max_threads: int = 32,
                 max_attempts: int = 3):
        self._rollout = _named(rollout_workers)
        self._pool = RoutingPool(self._rollout, call=lambda w, r: w.submit(r.request), max_attempts=max_attempts)
        self._trainers = _by_role(trainer_workers)
        self._inference = _by_role(inference_workers)
        self._weight_sync, self._export_weights = weight_sync, export_weights
        self._threads = cf.ThreadPoolExecutor(max_workers=max_threads, thread_name_prefix="rl-engine")
        self._done: "queue.Queue" = queue.Queue()
        self._inflight = 0
        self._policy_version = 0
        self._restored: Optional[dict] = None
        self._configured: dict = {}

    # ------------------------------------------------------------------ plumbing
    @property
    def policy_version(self) -> int:
        return self._policy_version

    @property
    def restored_checkpoint_metadata(self) -> Optional[dict]:
        return self._restored

    @property
    def rollout_pool(self) -> RoutingPool:
        return self._pool

    def follow_health(self, monitor, period_s: float = 1.0):
        """Keep the rollout rotation in step with a `HealthMonitor`: workers it reports silent, failed or stuck are taken
        out before a request has to fail on them, and put back when their reports are healthy again. Returns the event
        that stops the follower thread."""
        return self._pool.follow(monitor, period_s)

    async def _call(self, fn: Callable, *args, **kwargs):
        return await asyncio.get_running_loop().run_in_executor(self._threads, lambda: fn(*args, **kwargs))

    def _worker(self, table: dict, role, what: str):
        w = table.get(role_name(role))
        if w is None:
            raise ValueError(f"No {what} worker registered for role {role_name(role)}")
        return w

    # ------------------------------------------------------------------ rollouts
    def _build_rollout_requests(self, prompts: Sequence[Any], *, num_generations: int = 1, policy_version: int = 0,
                                generation_args: Optional[GenerationArgs] = None,
                                route_metadata: Optional[Mapping[str, Any]] = None, **kwargs: Any) -> list:
        base_meta = {**(route_metadata or {}), **(kwargs.get("metadata") or {})}
        base_gen = generation_args.as_kwargs() if generation_args else {}
        out: list = []
        for idx, p in enumerate(prompts):
            if isinstance(p, RolloutRequest):
                if not p.group_id:
                    raise ValueError(f"RolloutRequest at index {idx} (id={p.request_id!r}) lacks a group_id (the prompt id)")
                out.append(p)
                continue
            pid = _get(p, "prompt_id")
            if pid in (None, ""):
                raise ValueError(f"Prompt at index {idx} lacks 'prompt_id'. Every prompt dispatched to the engine must "
                                 "carry a unique 'prompt_id' (as an attribute or a dict key).")
            pid = str(pid)
            ids = _get(p, "prompt_ids", _get(p, "prompt_token_ids"))
            item_meta = dict(_get(p, "metadata") or {})
            for k in ("task", "env_config", "agent", "env", "agent_kwargs", "env_kwargs", "max_turns", "max_response_length"):
                if _get(p, k) is not None:
                    item_meta.setdefault(k, _get(p, k))       # what an episode worker builds its agent and environment from
            if ids is None:
                if "task" not in item_meta and "env_config" not in item_meta:
                    raise ValueError(f"Prompt {pid!r} has neither 'prompt_ids' (token ids) nor a 'task' for an episode worker")
                ids = []                                      # the agent renders the prompt from the task
            gen = {**base_gen, **dict(_get(p, "generation_kwargs") or {})}
            if _get(p, "max_response_length") is not None:
                gen["max_tokens"] = min(int(_get(p, "max_response_length")), int(gen.get("max_tokens", 1 << 30)))
            for g in range(num_generations):
                meta = {**base_meta, **item_meta, "prompt_id": pid, "group_index": g, "num_generations": num_generations}
                fields = {k: gen[k] for k in _REQUEST_FIELDS if gen.get(k) is not None}
                fields["seed"] = generate_vanilla_rollout_seed(pid, g) if fields.get("seed") is None else int(fields["seed"]) + g
                out.append(RolloutRequest(f"req_{pid}_g{g}_v{policy_version}", [int(t) for t in ids], group_id=pid,
                                          policy_version=policy_version, metadata=meta, **fields))
        for r in out:
            if r.metadata.get("lineage") is None:
                lin = LineageContext(tracking_id=r.request_id, parent_tracking_ids=[str(r.group_id)])
                lin.add_event("engine.dispatch", "rollout", {"policy_version": r.policy_version,
                                                             "group_index": r.metadata.get("group_index", 0)})
                r.metadata["lineage"] = lin
        return out

    def _run_one(self, req: RolloutRequest) -> None:
        try:
            resp = self._pool.submit(_Routed(req))
            if isinstance(resp, dict):
                resp = RolloutResponse(**resp)
            resp.metadata.setdefault("is_valid", True)
            for k in ("prompt_id", "group_index", "num_generations"):
                if k in req.metadata:
                    resp.metadata.setdefault(k, req.metadata[k])
        except Exception as e:
            log.error("rollout %s failed on every worker: %s", req.request_id, e)
            resp = RolloutResponse(req.request_id, [], None, None, policy_version=req.policy_version, finish_reason="error",
                                   group_id=req.group_id, metadata={**req.metadata, "is_valid": False, "error": repr(e)})
        self._done.put(resp)

    async def dispatch_rollout_requests(self, requests: Sequence[RolloutRequest]) -> list:
        requests = self._build_rollout_requests(requests)
        seen = set()
        for r in requests:
            if r.request_id in seen:
                raise ValueError(f"duplicate request_id {r.request_id!r} in one dispatch")
            seen.add(r.request_id)
        self._inflight += len(requests)
        for r in requests:
            self._threads.submit(self._run_one, r)
        return [r.request_id for r in requests]

    async def dispatch_rollouts(self, prompts: Sequence[Any], *, num_generations: int = 1, policy_version: int = 0,
                                generation_args: Optional[GenerationArgs] = None,
                                route_metadata: Optional[Mapping[str, Any]] = None, **kwargs: Any) -> list:
        return await self.dispatch_rollout_requests(self._build_rollout_requests(
            prompts, num_generations=num_generations, policy_version=policy_version, generation_args=generation_args,
            route_metadata=route_metadata, **kwargs))

    def _drain(self, timeout_s: float) -> list:
        out: list = []
        try:
            out.append(self._done.get(timeout=max(timeout_s, 0.0)) if timeout_s > 0 else self._done.get_nowait())
            while True:
                out.append(self._done.get_nowait())
        except queue.Empty:
            pass
        return out

    async def poll_rollouts(self, timeout_s: float = 1.0) -> list:
        got = self._drain(0.0)
        if not got and timeout_s > 0:
            # short naps keep the event loop's other stages running; with nothing in flight the call still takes its
            # time, so that a caller's polling loop cannot spin
            deadline = time.monotonic() + timeout_s
            while not got and time.monotonic() < deadline:
                await asyncio.sleep(0.002)
                got = self._drain(0.0)
        self._inflight -= len(got)
        return got

    async def generate(self, prompts: Sequence[Any], generation_args: Optional[GenerationArgs] = None,
                       route_metadata: Optional[Mapping[str, Any]] = None, **kwargs: Any) -> list:
        if kwargs:
            raise TypeError(f"Unexpected generate kwargs: {sorted(kwargs)}. Use generation_args=GenerationArgs(...) for sampling "
                            "parameters.")
        if not self._rollout:
            raise ValueError("DistributedRLEngine has no registered rollout workers.")
        reqs = self._build_rollout_requests(prompts, policy_version=self._policy_version, generation_args=generation_args,
                                            route_metadata=route_metadata)
        return list(await asyncio.gather(*(self._call(self._pool.submit, _Routed(r)) for r in reqs)))

    # ------------------------------------------------------------------ scoring, training
    async def score(self, role, items: Sequence[Any], op: str = "score", **kwargs: Any) -> list:
        return await self._call(self._worker(self._inference, role, "inference").submit, {"op": op, "items": items, **kwargs})

    async def per_token_logps(self, role, items: Any, op: str = "per_token_logps", **kwargs: Any) -> Any:
        w = self._inference.get(role_name(role))
        arrays = dict(items) if isinstance(items, Mapping) else {"items": items}
        if w is not None:
            return await self._call(w.submit, {"op": op, **arrays, **kwargs})
        w = self._trainers.get(role_name(role))
        if w is None:
            raise ValueError(f"No worker registered for per_token_logps with role {role_name(role)}")
        return await self._call(w.submit, {"op": "fwd_only", "batch": items, **kwargs})

    async def train_step(self, batch: Any, role=Role.ACTOR, accumulate_gradients: bool = False, apply_optimizer: bool = True,
                         **kwargs: Any) -> Any:
        w = self._worker(self._trainers, role, "trainer")
        arrays = getattr(batch, "arrays", batch)
        fb = await self._call(w.submit, {"op": "fwd_bwd", "batch": arrays, "is_last_microbatch": bool(apply_optimizer), **kwargs})
        if not apply_optimizer:
            return fb
        up = await self._call(w.submit, {"op": "update"})
        return {"fwd_bwd": fb, "updated": True, "train_step": up.get("step") if isinstance(up, Mapping) else up, "update": up,
                "accumulated": accumulate_gradients}

    async def get_metrics(self, role=Role.ACTOR, **kwargs: Any) -> Any:
        if role_name(role) == Role.ROLLOUT.value:
            if not self._rollout:
                raise ValueError("No rollout workers registered")
            return {"pool": self._pool.stats(), "inflight": self._inflight, "policy_version": self._policy_version}
        w = self._trainers.get(role_name(role)) or self._inference.get(role_name(role))
        if w is None:
            raise ValueError(f"No worker registered for role {role_name(role)}")
        return await self._call(w.submit, {"op": "get_metrics", **kwargs})

    def configure_worker(self, role=Role.ACTOR, *, algo: Any, assembler: Any, **kwargs: Any) -> None:
        """Checks that the role is served and keeps (algo, assembler) for it. A trainer worker of this package is built
        around a trainer that already holds its loss and input functions; an `algo` that offers `configure_trainer(worker)`
        is given the worker to install them."""
        name = role_name(role)
        if algo is None or assembler is None:
            raise ValueError(f"algo and assembler are required to configure the worker for role {name}")
        if name in (Role.ACTOR.value, Role.CRITIC.value):
            w = self._worker(self._trainers, role, "trainer")
            if hasattr(algo, "configure_trainer"):
                algo.configure_trainer(w)
        elif name == Role.ROLLOUT.value:
            if not self._rollout:
                raise ValueError("No rollout workers registered on engine.")
        elif name in (Role.REFERENCE.value, Role.REWARD.value):
            self._worker(self._inference, role, "inference")
        else:
            raise ValueError(f"Unsupported role for configure_worker: {name}")
        self._configured[name] = (algo, assembler, dict(kwargs))

    # ------------------------------------------------------------------ weights, checkpoints
    async def prepare_rollout_policy(self, role=Role.ACTOR, sync_weights: bool = True, policy_version: Optional[int] = None,
                                     **kwargs: Any) -> Optional[int]:
        self._worker(self._trainers, role, "trainer")
        if not sync_weights:
            return None
        return await self.sync_weights(role=role, policy_version=self._policy_version if policy_version is None else policy_version)

    def _push_weights(self, version: int) -> None:
        payload = self._export_weights() if self._export_weights is not None else None
        live = set(self._pool.live())
        ok, last = 0, None
        for name, w in self._rollout.items():
            if name not in live:
                continue
            try:
                w.sync_weights(version, payload)
                ok += 1
            except Exception as e:          # a worker that cannot take the weights must not serve stale ones: out of rotation
                last = e
                log.error("rollout worker %s failed to take policy version %d and is taken out of rotation: %s", name, version, e)
                self._pool.mark_down(name)
        if live and ok == 0:
            raise RuntimeError(f"no rollout worker took policy version {version}") from last

    async def sync_weights(self, role=Role.ACTOR, target_roles: Optional[Sequence[Any]] = None,
                           policy_version: Optional[int] = None, **kwargs: Any) -> int:
        version = self._policy_version + 1 if policy_version is None else int(policy_version)
        if self._weight_sync is not None:
            state = await self._call(self._weight_sync.run_round, version)
            if state != RoundState.COMMITTED:
                raise RuntimeError(f"weight sync round for policy_version={version} ended in state {getattr(state, 'value', state)}")
        else:
            await self._call(self._push_weights, version)
        self._policy_version = version
        return version

    async def save_checkpoint(self, role=Role.ACTOR, metadata: Any = None, **kwargs: Any) -> Any:
        w = self._worker(self._trainers, role, "trainer")
        return await self._call(w.submit, {"op": "save_checkpoint", "custom_metadata": dict(metadata or {}), "force": True, **kwargs})

    async def resume_from_checkpoint(self, role=Role.ACTOR, resync_rollout_weights: bool = True) -> int:
        self._restored = None
        w = self._worker(self._trainers, role, "trainer")
        got = await self._call(w.submit, {"op": "restore_checkpoint"})
        meta = got if isinstance(got, Mapping) else None
        if meta is None and got:
            try:
                meta = await self._call(w.submit, {"op": "restored_metadata"})
            except Exception:                                       # a trainer without metadata support: the step is all there is
                meta = None
            meta = dict(meta) if isinstance(meta, Mapping) else {"step": got}
        if not isinstance(meta, Mapping):
            return 0
        meta = dict(meta)
        try:
            opt_step = int(meta.get("step", 0) or 0)
            step = int(meta.get("global_step", opt_step) or 0)
        except (TypeError, ValueError):
            log.warning("restore_checkpoint returned a non-integer step %r; starting afresh", meta.get("global_step", meta.get("step")))
            return 0
        if step <= 0:
            return 0
        self._restored = meta
        recorded = meta.get("policy_version")
        off_policy = "committed_prompt_ids" in meta or "skipped_prompt_ids" in meta
        if off_policy and recorded is not None:
            version = int(recorded)
        else:
            version = step
            if recorded is not None and int(recorded) != step:
                log.warning("checkpoint recorded policy_version=%s inside a step; resuming at the step boundary %d", recorded, step)
        self._policy_version = version
        if resync_rollout_weights:
            synced = await self.sync_weights(role=role, policy_version=version)
            if synced != version:
                raise RuntimeError(f"resumed policy_version={version} does not match the synced version {synced}")
        else:
            log.warning("resync_rollout_weights is False: rollout workers keep their weights instead of checkpoint version %d", version)
        return step

    async def close(self) -> None:
        self._threads.shutdown(wait=False, cancel_futures=True)
