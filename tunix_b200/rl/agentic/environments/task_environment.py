"""Single-turn task environment: one question, the response is scored by a reward function
(tunix/rl/agentic/environments/task_environment.py)."""
from __future__ import annotations

from typing import Any, Callable, Optional

from ..rewards.reward import get_reward_fn
from .base_environment import BaseTaskEnv


class TaskEnvironment(BaseTaskEnv):
    def __init__(self, task: Any = None, reward_fn: Optional[Callable] = None, max_steps: int = 1, **kwargs):
        super().__init__(task, max_steps, **kwargs)
        self.reward_fn = get_reward_fn(reward_fn) if isinstance(reward_fn, str) else (reward_fn or get_reward_fn("zero"))

    def _initial_observation(self):
        return self.task if isinstance(self.task, dict) else {"question": self.task}

    def _step_impl(self, action):
        out = self.reward_fn(task=self.task, action=action)
        return {}, float(out.reward), True, {"response": action, "metadata": out.metadata}
