"""Core data types of the agent system (tunix/rl/agentic/agents/agent_types.py)."""
from __future__ import annotations

import dataclasses
import enum
from typing import Any, Optional

import numpy as np

UNSET_ROUTED_EXPERT = -1


@dataclasses.dataclass(kw_only=True)
class Action:
    action: Any = None


@dataclasses.dataclass(kw_only=True)
class Step:
    chat_completions: list = dataclasses.field(default_factory=list)
    thought: str = ""
    action: Optional[Action] = None
    observation: Any = None
    model_response: str = ""
    info: dict = dataclasses.field(default_factory=dict)
    reward: float = 0.0
    done: bool = False
    mc_return: float = 0.0
    assistant_tokens: Optional[np.ndarray] = None
    assistant_masks: Optional[np.ndarray] = None
    env_tokens: Optional[np.ndarray] = None
    env_masks: Optional[np.ndarray] = None
    logprobs: Optional[np.ndarray] = None
    policy_version: Optional[Any] = None          # version of the weights this step's tokens were sampled with
    routed_experts: Optional[np.ndarray] = None   # [tokens of the call, num_layers, top_k] when the sampler reports it


class TrajectoryStatus(enum.Enum):
    SUCCEEDED = enum.auto()
    RUNNING = enum.auto()
    MAX_STEPS_REACHED = enum.auto()
    MAX_CONTEXT_LIMIT_REACHED = enum.auto()
    TIMEOUT = enum.auto()
    ENV_TIMEOUT = enum.auto()
    FAILED = enum.auto()
    CANCELLED = enum.auto()
    PARTIAL = enum.auto()          # handed back unfinished by collect(max_new_steps=...); resume() continues it


INVALID_TRAJECTORY_STATUSES = frozenset({TrajectoryStatus.FAILED, TrajectoryStatus.TIMEOUT,
                                         TrajectoryStatus.ENV_TIMEOUT, TrajectoryStatus.CANCELLED})


@dataclasses.dataclass(kw_only=True)
class Trajectory:
    task: Any = None
    steps: list = dataclasses.field(default_factory=list)
    step_idx: int = -1
    reward: float = 0.0
    status: TrajectoryStatus = TrajectoryStatus.RUNNING
    masked_out: Optional[bool] = None
    env_time: dict = dataclasses.field(default_factory=dict)


@dataclasses.dataclass(kw_only=True)
class TrajectoryItem:
    """What travels from the rollout pipeline to the learner: one finished episode of one (prompt, generation) pair."""
    pair_index: int
    group_id: Any
    episode_id: int
    start_step: int
    traj: Any
    metadata: dict = dataclasses.field(default_factory=dict)


def is_valid_trajectory_dict(traj: Any) -> bool:
    if not isinstance(traj, dict):
        return False
    status = traj.get("status")
    if isinstance(status, str):
        status = TrajectoryStatus.__members__.get(status.upper(), status)
    if status in INVALID_TRAJECTORY_STATUSES:
        return False
    masks = traj.get("conversation_masks")
    return True if masks is None else bool(np.sum(masks) > 0)
