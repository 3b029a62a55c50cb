"""Gym-like environment interface with async variants (tunix/rl/agentic/environments/base_environment.py)."""
from __future__ import annotations

import abc
import asyncio
from typing import Any


class BaseTaskEnv(abc.ABC):
    def __init__(self, task: Any = None, max_steps: int = 1, **kwargs):
        self.task = task
        self.max_steps = max_steps
        self.step_count = 0
        self.extra_kwargs = kwargs

    def reset(self):
        self.step_count = 0
        return self._initial_observation(), {}

    def step(self, action: Any):
        self.step_count += 1
        obs, reward, done, info = self._step_impl(action)
        if self.step_count >= self.max_steps:
            done = True
        return obs, reward, done, info

    async def reset_async(self):
        return await asyncio.get_running_loop().run_in_executor(None, self.reset)

    async def step_async(self, action: Any):
        return await asyncio.get_running_loop().run_in_executor(None, lambda: self.step(action))

    def close(self) -> None:
        pass

    @abc.abstractmethod
    def _initial_observation(self) -> Any: ...

    @abc.abstractmethod
    def _step_impl(self, action: Any): ...

    @classmethod
    def from_dict(cls, d: dict):
        return cls(**d)
