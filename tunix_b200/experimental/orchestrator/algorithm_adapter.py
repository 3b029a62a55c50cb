"""What differs between RL algorithms on the distributed path
(tunix/experimental/orchestrator/algorithm_adapter.py:123-480): how one prompt's responses become trainer payloads.

`GRPOAdapter`  group-relative advantages (GRPO, Dr. GRPO without the std division, RLOO leave-one-out baseline),
               one scalar per response broadcast over its tokens; groups whose rewards are all equal are dropped.
`PPOAdapter`   per-token advantages from a critic: the scalar reward lands on the last token, an optional KL
               penalty against reference log-probs is charged per token, values come from `value_fn` (usually a
               critic worker's `fwd_only`), GAE runs backwards over the response
               (`rl.algo_core.compute_gae_advantages`), and the payload carries `returns` and `values` (the critic's
               predictions at rollout time) for the value loss.

Both produce `RLTrainerPayload`s whose `example` dict is what `BatchAssembler` pads or packs."""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Optional, Sequence

import numpy as np

from ..common.datatypes import RLTrainerPayload


def env_reward(item: dict, r) -> float:
    """The reward an episode's environment gave (multi-turn workers report it as `trajectory_reward`)."""
    return float((r.metadata or {}).get("trajectory_reward", 0.0))


def _base_example(item: dict, r, advantages: np.ndarray) -> dict:
    """A response of a multi-turn worker brings its own prompt (rendered by the agent) and a mask that leaves the
    environment's tokens out of the loss; a single-call response uses the item's prompt and trains on every token."""
    n = len(r.tokens)
    md = r.metadata or {}
    mask = np.asarray(md["conversation_masks"], np.float32) if md.get("conversation_masks") is not None else np.ones(n, np.float32)
    if md.get("masked_out"):
        mask = np.zeros(n, np.float32)
    prompt = md["prompt_token_ids"] if md.get("prompt_token_ids") else item["prompt_ids"]
    ex = {"prompt_ids": np.asarray(prompt, np.int32), "completion_ids": np.asarray(r.tokens, np.int32),
          "completion_mask": mask, "advantages": np.asarray(advantages, np.float32),
          "lineage": md.get("lineage"), "prompt_id": str(item.get("prompt_id", ""))}
    if r.logprobs is not None:
        ex["old_per_token_logps"] = np.asarray(r.logprobs, np.float32)
    return ex


@dataclasses.dataclass
class GRPOAdapter:
    reward_fn: Callable[[dict, Any], float]
    estimator: str = "grpo"                                 # "grpo" | "drgrpo" | "rloo"
    drop_uniform_groups: bool = True
    advantage_fn: Optional[Callable[[np.ndarray], np.ndarray]] = None

    def advantages(self, rewards: np.ndarray) -> np.ndarray:
        r = np.asarray(rewards, np.float32)
        if self.advantage_fn is not None:
            return np.asarray(self.advantage_fn(r), np.float32)
        if self.estimator == "grpo":
            return ((r - r.mean()) / (r.std() + 1e-6)).astype(np.float32)
        if self.estimator == "drgrpo":
            return (r - r.mean()).astype(np.float32)
        if self.estimator == "rloo":
            n = len(r)
            if n < 2:
                raise ValueError("rloo needs at least two responses per prompt")
            return (r - (r.sum() - r) / (n - 1)).astype(np.float32)
        raise ValueError(f"unknown estimator {self.estimator!r}")

    def create_payloads(self, item: dict, responses: Sequence) -> list:
        rewards = np.asarray([self.reward_fn(item, r) for r in responses], np.float32)
        if self.drop_uniform_groups and float(rewards.std()) == 0.0:
            return []
        adv = self.advantages(rewards)
        return [RLTrainerPayload(_base_example(item, r, np.full(len(r.tokens), a, np.float32)), policy_version=r.policy_version,
                                 group_id=r.group_id, reward=float(rew)) for r, a, rew in zip(responses, adv, rewards)]


@dataclasses.dataclass
class PPOAdapter:
    reward_fn: Callable[[dict, Any], float]
    value_fn: Callable[[Sequence[int], Sequence[int]], Sequence[float]]        # (prompt ids, completion ids) -> V per completion token
    ref_logps_fn: Optional[Callable[[Sequence[int], Sequence[int]], Sequence[float]]] = None
    gamma: float = 1.0
    gae_lambda: float = 0.95
    kl_coef: float = 0.0
    whiten: bool = True
    drop_uniform_groups: bool = False                       # a critic learns from uniform groups too

    def create_payloads(self, item: dict, responses: Sequence) -> list:
        import torch
        from ...rl.algo_core import compute_gae_advantages
        if not responses:
            return []
        scores = np.asarray([self.reward_fn(item, r) for r in responses], np.float32)
        T = max(len(r.tokens) for r in responses)
        rew, val, mask = (np.zeros((len(responses), T), np.float32) for _ in range(3))
        for i, r in enumerate(responses):
            n = len(r.tokens)
            if n == 0:
                continue
            mask[i, :n] = 1.0
            val[i, :n] = np.asarray(self.value_fn(item["prompt_ids"], r.tokens), np.float32)[:n]
            if self.kl_coef and self.ref_logps_fn is not None and r.logprobs is not None:
                ref = np.asarray(self.ref_logps_fn(item["prompt_ids"], r.tokens), np.float32)[:n]
                rew[i, :n] -= self.kl_coef * (np.asarray(r.logprobs, np.float32)[:n] - ref)
            rew[i, n - 1] += scores[i]
        adv, ret = compute_gae_advantages(torch.from_numpy(rew), torch.from_numpy(val), torch.from_numpy(mask),
                                          self.gamma, self.gae_lambda, whiten=self.whiten and mask.sum() > 1)
        adv, ret = adv.numpy(), ret.numpy()
        out = []
        for i, r in enumerate(responses):
            n = len(r.tokens)
            ex = _base_example(item, r, adv[i, :n])
            ex["returns"], ex["values"] = ret[i, :n].astype(np.float32), val[i, :n].copy()
            out.append(RLTrainerPayload(ex, policy_version=r.policy_version, group_id=r.group_id, reward=float(scores[i])))
        return out
