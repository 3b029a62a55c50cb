"""One rollout episode with lifecycle controls (tunix/experimental/rollout/collector.py:34-511).

`TrajectoryCollectorEngine` wraps the multi-turn episode loop of `rl.agentic.trajectory.TrajectoryCollectEngine` for
the distributed rollout workers:

* every model call goes to an asynchronous sampler (`experimental.rollout.sampler.AsyncSampler`) with the request's
  sampling settings; the token budget of a call is the smaller of the episode's remaining budget and the request's own
  limit; a sampler that needs a seed gets a deterministic one from (prompt id, index in the group);
* `pause()` holds the episode before its next model call (weight sync), `resume()` lets it go on, `cancel()` marks it
  cancelled; the policy version of every turn is recorded (a paused episode may continue under newer weights);
* the finished episode comes back as an `agent_types.TrajectoryItem` whose metadata carries request-scoped facts only
  (prompt id, group index, status, policy versions) plus the response-budget facts `raw_length` / `clipped`
  (`response_budget_facts`): truncated = reached the budget without ending on a configured stop token.
"""
from __future__ import annotations

import asyncio
import logging
import zlib
from typing import Callable, Collection, Optional, Sequence

import numpy as np

from ...rl.agentic.agents import agent_types
from ...rl.agentic.trajectory.trajectory_collect_engine import TrajectoryCollectEngine
from . import sampler as sampler_lib

log = logging.getLogger(__name__)
_DEFAULT_EPISODE_TIMEOUT_SECS = 600.0


def generate_vanilla_rollout_seed(prompt_id, group_index: int = 0) -> int:
    """Deterministic 31-bit seed of one rollout: (crc32(prompt id) + index in the group) mod 2^31, so the G rollouts
    of a prompt differ and a re-run of the same request samples the same tokens."""
    return ((zlib.crc32(str(prompt_id).encode("utf-8")) & 0x7FFFFFFF) + int(group_index)) & 0x7FFFFFFF


def response_budget_facts(response_tokens: Sequence[int], max_response_length: int, eos_ids: Collection[int]):
    """(raw_length, clipped): `clipped` is True when the response reached `max_response_length` tokens without ending
    on one of `eos_ids`; `raw_length` is clamped to the budget."""
    if max_response_length <= 0:
        raise ValueError(f"max_response_length must be positive, got {max_response_length}")
    n = len(response_tokens)
    stopped = 0 < n <= max_response_length and int(response_tokens[-1]) in eos_ids
    return min(n, max_response_length), (n >= max_response_length and not stopped)


class TrajectoryCollectorEngine:
    """`request`: an object with `prompt_id`, `group_index`, `generation_kwargs` (temperature, top_p, top_k, seed,
    max_tokens), `max_turns`, `max_response_length`, `target_policy_version`, `metadata` (optional `episode_timeout`,
    `overlong_filter`). `sampler`: an `AsyncSampler`. `policy_version_fn()` reports the sampler's current weights."""

    def __init__(self, traj_id: str, request, sampler, env_client, agent, tokenizer, chat_parser=None,
                 eos_ids: Optional[Collection[int]] = None, partial_rollout: bool = False,
                 policy_version_fn: Optional[Callable[[], int]] = None, needs_seed: bool = True):
        if sampler is None or env_client is None or agent is None or tokenizer is None:
            raise ValueError("TrajectoryCollectorEngine needs a sampler, an environment, an agent and a tokenizer")
        self.traj_id, self.request = traj_id, request
        self.sampler, self.env, self.agent = sampler, env_client, agent
        self.tokenizer, self.chat_parser = tokenizer, chat_parser
        self.partial_rollout = bool(partial_rollout)
        self.needs_seed = needs_seed
        self._policy_version_fn = policy_version_fn
        self.is_paused = self.is_cancelled = self.is_done = False
        self._unpaused = asyncio.Event()
        self._unpaused.set()
        self._turn_policy_versions: list = []
        self._inner: Optional[TrajectoryCollectEngine] = None
        self.max_response_length = getattr(request, "max_response_length", None)
        self.eos_ids = frozenset(int(t) for t in (eos_ids or ()))
        md = getattr(request, "metadata", None) or {}
        timeout = md.get("episode_timeout")
        self.episode_timeout = float(_DEFAULT_EPISODE_TIMEOUT_SECS if timeout is None else timeout)
        if self.episode_timeout <= 0:
            raise ValueError("episode_timeout must be positive.")
        of = md.get("overlong_filter")
        if of is not None and not isinstance(of, bool):
            raise TypeError(f"overlong_filter must be a boolean, got {type(of).__name__}: {of!r}.")
        self.overlong_filter = bool(of)

    # ------------------------------------------------------------------ one model call
    async def _model_call(self, chat_completions=None, prompt_token_ids=None, max_tokens=None, **kwargs) -> dict:
        await self._unpaused.wait()                               # a paused episode stops before its next call
        gen = dict(getattr(self.request, "generation_kwargs", None) or {})
        gen.update(kwargs)
        own = gen.pop("max_generation_steps", None)
        own = own if own is not None else gen.get("max_tokens")
        limits = [x for x in (max_tokens, own) if x is not None]
        if not limits:
            raise ValueError("no token limit: give the request max_response_length or generation_kwargs max_tokens")
        seed = gen.get("seed")
        if seed is None and self.needs_seed:
            pid = getattr(self.request, "prompt_id", None)
            if pid is None:
                raise ValueError("the sampler needs a seed: give generation_kwargs['seed'] or a prompt_id")
            seed = generate_vanilla_rollout_seed(pid, getattr(self.request, "group_index", 0))
        req_version = int(getattr(self.request, "target_policy_version", 0) or 0)
        version = max(req_version, int(self._policy_version_fn())) if self._policy_version_fn else req_version
        self._turn_policy_versions.append(version)
        if prompt_token_ids is None:
            text = self.chat_parser.parse(chat_completions, add_generation_prompt=True, is_first_msg=True) \
                if (self.chat_parser is not None and not isinstance(chat_completions, str)) else str(chat_completions)
            prompt_token_ids = list(self.tokenizer.encode(text))
        params = sampler_lib.SamplingParams(max_tokens=int(min(limits)), temperature=gen.get("temperature", 0.0),
                                            top_p=gen.get("top_p"), top_k=gen.get("top_k"), seed=seed,
                                            return_logprobs=gen.get("return_logprobs", True))
        sreq = sampler_lib.SamplingRequest(request_id=self.traj_id, prompt_token_ids=list(prompt_token_ids),
                                           sampling_params=params, route_key=str(getattr(self.request, "prompt_id", "")))
        res = (await self.sampler.sample([sreq]))[0]
        if getattr(res, "error", None) is not None:
            raise res.error
        toks = list(res.token_ids)
        text = res.text if res.text is not None else self.tokenizer.decode(toks)
        return {"text": text, "tokens": toks, "logprobs": res.logprobs if res.logprobs is not None else [0.0] * len(toks),
                "policy_version": version}

    # ------------------------------------------------------------------ episode
    async def run_episode(self) -> agent_types.TrajectoryItem:
        self._turn_policy_versions = []
        self._inner = TrajectoryCollectEngine(
            self.agent, self.env, model_call=self._model_call, tokenizer=self.tokenizer, chat_parser=self.chat_parser,
            max_steps=int(getattr(self.request, "max_turns", 10)), timeout=self.episode_timeout,
            max_response_length=self.max_response_length, overlong_filter=self.overlong_filter)
        traj = await self._inner.collect(mode="Token")
        if self.is_cancelled:
            traj["status"] = agent_types.TrajectoryStatus.CANCELLED
        if isinstance(traj, dict) and self._turn_policy_versions:
            traj["policy_version"] = int(self._turn_policy_versions[0])
            traj["policy_versions"] = list(self._turn_policy_versions)
        self.is_done = True
        return self._to_item(traj)

    def _annotate_response_budget(self, traj: dict, metadata: dict) -> None:
        """`raw_length` / `clipped` when a budget was enforced, a stop set is known and there is a token stream;
        left unset otherwise, so that a consumer can tell "not truncated" from "unknown"."""
        if not self.max_response_length or self.max_response_length <= 0 or not self.eos_ids:
            return
        toks = traj.get("conversation_tokens")
        if toks is None:
            return
        metadata["raw_length"], metadata["clipped"] = response_budget_facts(list(np.asarray(toks)), self.max_response_length,
                                                                            self.eos_ids)

    def _to_item(self, traj: dict) -> agent_types.TrajectoryItem:
        if not isinstance(traj, dict):
            raise TypeError(f"expected a token-mode trajectory dict, got {type(traj).__name__}")
        md = dict(getattr(self.request, "metadata", None) or {})
        md["prompt_id"] = getattr(self.request, "prompt_id", None)
        md["group_index"] = getattr(self.request, "group_index", 0)
        md["status"] = traj.get("status", "")
        versions = self._turn_policy_versions or [int(getattr(self.request, "target_policy_version", 0) or 0)]
        md["policy_version"], md["policy_versions"] = int(versions[0]), list(versions)
        if md.pop("record_episode_summary", False):
            steps = self.agent.trajectory.steps
            blocked = [s.info or {} for s in steps if (getattr(s, "info", None) or {}).get("guard_blocked")]
            traj["episode_summary"] = {"num_steps": len(steps), "guard_blocked_steps": len(blocked),
                                       "guard_reasons": sorted({str(b.get("guard_reason") or "unknown") for b in blocked})}
        self._annotate_response_budget(traj, md)
        return agent_types.TrajectoryItem(pair_index=md["group_index"], group_id=md["prompt_id"], episode_id=0, start_step=0,
                                          traj=traj, metadata=md)

    # ------------------------------------------------------------------ lifecycle
    def pause(self) -> None:
        self.is_paused = True
        self._unpaused.clear()

    def resume(self) -> None:
        self.is_paused = False
        self._unpaused.set()

    def cancel(self) -> None:
        """Mark the episode cancelled; a paused episode is released so that its task can end."""
        if self.is_done:
            return
        self.is_cancelled = True
        if self.agent is not None:
            self.agent.trajectory.status = agent_types.TrajectoryStatus.CANCELLED
        self._unpaused.set()
