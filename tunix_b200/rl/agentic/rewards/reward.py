"""Reward registry for agentic environments (tunix/rl/agentic/rewards/reward.py, reward_types.py)."""
from __future__ import annotations

import dataclasses
import re
from typing import Any, Callable


@dataclasses.dataclass
class RewardOutput:
    reward: float
    metadata: dict = dataclasses.field(default_factory=dict)


_REGISTRY: dict = {}


def register(name: str):
    def deco(fn):
        _REGISTRY[name] = fn
        return fn
    return deco


def get_reward_fn(name_or_fn) -> Callable:
    if callable(name_or_fn):
        return name_or_fn
    if name_or_fn not in _REGISTRY:
        raise ValueError(f"unknown reward function {name_or_fn!r}; known: {sorted(_REGISTRY)}")
    return _REGISTRY[name_or_fn]


@register("zero")
def zero_reward(task: Any, action: Any) -> RewardOutput:
    return RewardOutput(0.0)


@register("exact_match")
def exact_match(task: Any, action: Any) -> RewardOutput:
    gold = str(task.get("answer", task.get("ground_truth", ""))).strip() if isinstance(task, dict) else ""
    return RewardOutput(1.0 if str(action).strip() == gold else 0.0, {"gold": gold})


@register("calculate")
def calculate_reward(task: Any, action: Any) -> RewardOutput:
    """Numeric answer check tolerant to surrounding text."""
    gold = task.get("answer") if isinstance(task, dict) else None
    nums = re.findall(r"-?\d+\.?\d*", str(action))
    try:
        ok = bool(nums) and gold is not None and abs(float(nums[-1]) - float(gold)) < 1e-6
    except ValueError:
        ok = False
    return RewardOutput(1.0 if ok else 0.0)


def combine_rewards(weights: dict) -> Callable:
    """Weighted sum of registered rewards: {name: weight}."""
    fns = {get_reward_fn(n): w for n, w in weights.items()}

    def combined(task, action):
        total, meta = 0.0, {}
        for fn, w in fns.items():
            o = fn(task=task, action=action)
            total += w * o.reward
            meta[getattr(fn, "__name__", "fn")] = o.reward
        return RewardOutput(total, meta)
    return combined
