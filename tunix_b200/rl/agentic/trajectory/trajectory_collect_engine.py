"""One agent/environment episode: reset -> (model call -> agent update -> env step)* with budgets
(tunix/rl/agentic/trajectory/trajectory_collect_engine.py:48-1357).

Limits: per-episode wall-clock `timeout`, `max_steps`, `max_response_length` tokens over all assistant and
environment turns (context limit), per env-step timeout. Every turn records assistant token ids, their
sampled log-probs and masks (assistant 1 / environment 0); later turns are prompted with the recorded ids
(exact token continuity). Monte-Carlo returns are filled at the end. Output modes: "Trajectory" (objects),
"Token" (flattened arrays for training), "Steps", "Conversation".

Also (tunix/rl/agentic/trajectory/trajectory_collect_engine.py:407-470,877-...):
* routed experts: a model call that reports `routed_experts` (mixture-of-experts router replay) has them stored on
  its step and concatenated, per token of the conversation, in the "Token" output;
* context window: with `max_context_tokens` the episode ends (MAX_CONTEXT_LIMIT_REACHED) before a model call whose
  prompt would not leave room for a reply;
* partial rollouts: `collect(..., max_new_steps=k)` stops after k further turns with status PARTIAL and keeps agent,
  environment and token context alive; `resume()` continues the same episode (typically after a weight sync; every
  step records the `policy_version` its tokens were sampled with)."""
from __future__ import annotations

import asyncio
import time
from typing import Any, Awaitable, Callable, Optional

import numpy as np

from ..agents.agent_types import Trajectory, TrajectoryStatus
from ..utils import concat_conversation


class _EpisodeTimeout(Exception):
    """The episode's wall-clock budget ran out inside a model call or an environment step."""


class TrajectoryCollectEngine:
    def __init__(self, agent, env, *, model_call: Callable[..., Awaitable[dict]], tokenizer=None, chat_parser=None,
                 max_steps: int = 10, gamma: float = 1.0, timeout: float = 600.0, env_step_timeout: Optional[float] = None,
                 max_response_length: Optional[int] = None, final_reward_fn: Optional[Callable] = None,
                 overlong_filter: bool = False, max_context_tokens: Optional[int] = None):
        self.agent, self.env = agent, env
        self.model_call = model_call
        self.tokenizer, self.chat_parser = tokenizer, chat_parser
        self.max_steps, self.gamma, self.timeout = max_steps, gamma, timeout
        self.env_step_timeout = env_step_timeout
        self.max_response_length = max_response_length
        self.final_reward_fn = final_reward_fn
        self.overlong_filter = overlong_filter
        self.max_context_tokens = max_context_tokens
        self._used = 0
        self._started = False
        self._start = 0.0
        self._prompt_tokens: Optional[np.ndarray] = None
        self._context: list = []

    # --------------------------------------------------------------- episode
    async def collect(self, mode: str = "Trajectory", max_new_steps: Optional[int] = None):
        """Run the episode (or, after a PARTIAL return, continue it). `max_new_steps`: hand the episode back after
        this many further turns if it is not over by then."""
        traj = self.agent.trajectory
        partial = False
        try:
            if not self._started:
                await self._reset()
                self._started, self._used = True, 0
            traj = self.agent.trajectory
            traj.status = TrajectoryStatus.RUNNING
            new_steps = 0
            while True:
                if len(traj.steps) >= self.max_steps:
                    traj.status = TrajectoryStatus.MAX_STEPS_REACHED
                    break
                if max_new_steps is not None and new_steps >= max_new_steps:
                    traj.status, partial = TrajectoryStatus.PARTIAL, True
                    break
                if time.monotonic() - self._start > self.timeout:
                    traj.status = TrajectoryStatus.TIMEOUT
                    break
                if self.max_context_tokens is not None and self._prompt_tokens is not None and \
                        len(self._context) + 1 > self.max_context_tokens:
                    traj.status = TrajectoryStatus.MAX_CONTEXT_LIMIT_REACHED     # no room left for a reply
                    break
                done, n_tok = await self._one_step(traj, self._used)
                self._used += n_tok
                new_steps += 1
                if done:
                    traj.status = TrajectoryStatus.SUCCEEDED
                    break
                if self.max_response_length is not None and self._used >= self.max_response_length:
                    traj.status = TrajectoryStatus.MAX_CONTEXT_LIMIT_REACHED
                    break
        except asyncio.CancelledError:
            traj.status = TrajectoryStatus.CANCELLED
            raise
        except _EpisodeTimeout:
            traj.status = TrajectoryStatus.TIMEOUT
        except asyncio.TimeoutError:
            traj.status = TrajectoryStatus.ENV_TIMEOUT
        except Exception as e:  # model, env or reward failure: the episode is invalid, the pipeline goes on
            traj.status = TrajectoryStatus.FAILED
            traj.env_time["error"] = f"{type(e).__name__}: {e}"
        finally:
            if not partial:
                try:
                    t0 = time.monotonic()
                    self.env.close()
                    traj.env_time["close_latency"] = time.monotonic() - t0
                except Exception:
                    pass
        if not partial:
            self._finalize(traj)
        return self._format(traj, mode)

    async def resume(self, mode: str = "Trajectory", max_new_steps: Optional[int] = None):
        """Continue an episode that `collect(max_new_steps=...)` handed back as PARTIAL."""
        if not self._started or self.agent.trajectory.status != TrajectoryStatus.PARTIAL:
            raise RuntimeError("resume() continues an episode that collect() returned as PARTIAL")
        return await self.collect(mode, max_new_steps)

    async def _reset(self):
        self._start = time.monotonic()
        self.agent.reset()
        t0 = time.monotonic()
        obs, info = await self.env.reset_async()
        self.agent.trajectory.env_time["reset_latency"] = time.monotonic() - t0
        self.agent.trajectory.env_time["step_latency"] = []
        self.agent.trajectory.task = getattr(self.env, "task", None)
        await self.agent.update_from_env_async(obs, 0.0, False, info)
        self._context = []
        self._prompt_tokens = None

    def _render_prompt(self, new_messages_only: bool) -> list:
        msgs = self.agent.chat_completions
        if self.chat_parser is not None:
            text = self.chat_parser.parse(msgs, add_generation_prompt=True)
        elif self.tokenizer is not None and hasattr(self.tokenizer, "apply_chat_template"):
            text = self.tokenizer.apply_chat_template(msgs, add_generation_prompt=True, tokenize=False)
        else:
            text = "\n".join(str(m["content"]) for m in msgs)
        return list(self.tokenizer.encode(text)) if self.tokenizer is not None else []

    async def _one_step(self, traj: Trajectory, used_tokens: int):
        traj.step_idx += 1
        if self._prompt_tokens is None:
            self._prompt_tokens = np.asarray(self._render_prompt(False), np.int64)
            self._context = list(self._prompt_tokens)
        budget = None if self.max_response_length is None else max(self.max_response_length - used_tokens, 1)
        # the model call may take no longer than what is left of the episode's budget; a call that is cut off is
        # cancelled (its client sees CancelledError) and the episode ends as TIMEOUT
        remaining = self.timeout - (time.monotonic() - self._start)
        try:
            out = await asyncio.wait_for(self.model_call(chat_completions=self.agent.chat_completions,
                                                         prompt_token_ids=list(self._context), max_tokens=budget),
                                         max(remaining, 1e-3))
        except asyncio.TimeoutError:
            raise _EpisodeTimeout() from None
        action = await self.agent.update_from_model_async(out["text"])
        step = self.agent.get_current_step()
        a_tok = np.asarray(out.get("tokens", []), np.int64)
        step.assistant_tokens = a_tok
        step.assistant_masks = np.ones(len(a_tok), np.int32)
        step.logprobs = np.asarray(out.get("logprobs", np.zeros(len(a_tok))), np.float32)
        step.policy_version = out.get("policy_version")
        step.routed_experts = None if out.get("routed_experts") is None else np.asarray(out["routed_experts"], np.int16)
        self._context.extend(a_tok.tolist())
        t0 = time.monotonic()
        coro = self.env.step_async(action.action)
        remaining = self.timeout - (time.monotonic() - self._start)
        limit = min(self.env_step_timeout, remaining) if self.env_step_timeout else remaining
        try:
            obs, reward, done, info = await asyncio.wait_for(coro, max(limit, 1e-3))
        except asyncio.TimeoutError:
            if self.env_step_timeout and self.env_step_timeout <= remaining:
                raise                                        # the environment's own limit: ENV_TIMEOUT
            raise _EpisodeTimeout() from None
        traj.env_time["step_latency"].append(time.monotonic() - t0)
        n_before = len(self.agent.chat_completions)
        await self.agent.update_from_env_async(obs, reward, done, info)
        env_tok = np.zeros(0, np.int64)
        new_msgs = self.agent.chat_completions[n_before:]
        if new_msgs and not done and self.tokenizer is not None:
            if self.chat_parser is not None:
                text = self.chat_parser.parse(new_msgs, add_generation_prompt=True, is_first_msg=False)
            else:
                text = "\n".join(str(m["content"]) for m in new_msgs)
            env_tok = np.asarray(self.tokenizer.encode(text), np.int64)
            self._context.extend(env_tok.tolist())
        step.env_tokens = env_tok
        step.env_masks = np.zeros(len(env_tok), np.int32)
        return done, len(a_tok) + len(env_tok)

    def _finalize(self, traj: Trajectory) -> None:
        g = 0.0
        for s in reversed(traj.steps):
            g = s.reward + self.gamma * g
            s.mc_return = g
        traj.reward = float(sum(s.reward for s in traj.steps))
        if self.final_reward_fn is not None and traj.steps:
            extra = self.final_reward_fn(traj.task, traj.steps[-1].model_response)
            traj.reward += float(getattr(extra, "reward", extra))
        traj.masked_out = bool(self.overlong_filter and traj.status in (TrajectoryStatus.MAX_CONTEXT_LIMIT_REACHED,
                                                                         TrajectoryStatus.MAX_STEPS_REACHED,
                                                                         TrajectoryStatus.TIMEOUT))

    def _format(self, traj: Trajectory, mode: str):
        if mode == "Trajectory":
            return traj
        if mode == "Steps":
            return traj.steps
        if mode == "Conversation":
            return self.agent.chat_completions
        if mode == "Token":
            toks, masks, lps = concat_conversation(self._prompt_tokens, traj.steps)
            if traj.masked_out:
                masks = np.zeros_like(masks)
            routed = [getattr(s_, "routed_experts", None) for s_ in traj.steps]
            versions = [getattr(s_, "policy_version", None) for s_ in traj.steps]
            return {"prompt_tokens": self._prompt_tokens if self._prompt_tokens is not None else np.zeros(0, np.int64),
                    "conversation_tokens": toks, "conversation_masks": masks, "old_logprobs": lps,
                    "trajectory_reward": traj.reward, "status": traj.status, "masked_out": traj.masked_out,
                    "policy_version": min((v for v in versions if v is not None), default=None),
                    "policy_versions": versions, "num_turns": len(traj.steps),
                    # one routing array per model call (None when any call did not report its routing)
                    "routed_experts": routed if routed and all(r is not None for r in routed) else None}
        raise ValueError(f"unknown output mode {mode!r}")
