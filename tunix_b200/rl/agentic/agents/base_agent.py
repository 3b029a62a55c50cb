"""Agent base classes (tunix/rl/agentic/agents/base_agent.py): `LLMBaseAgent` (protocol) and
`ConversationAgentBase` (chat history + trajectory bookkeeping)."""
from __future__ import annotations

import abc
import asyncio
from typing import Any

from .agent_types import Action, Step, Trajectory


class LLMBaseAgent(abc.ABC):
    @property
    @abc.abstractmethod
    def chat_completions(self) -> list: ...

    @property
    @abc.abstractmethod
    def trajectory(self) -> Trajectory: ...

    @abc.abstractmethod
    def update_from_env(self, observation: Any, reward: float, done: bool, info: dict, **kwargs) -> None: ...

    async def update_from_env_async(self, *args, **kwargs) -> None:
        return await asyncio.get_running_loop().run_in_executor(None, lambda: self.update_from_env(*args, **kwargs))

    @abc.abstractmethod
    def update_from_model(self, response: str, **kwargs) -> Action: ...

    async def update_from_model_async(self, response: str, **kwargs) -> Action:
        return self.update_from_model(response, **kwargs)

    @abc.abstractmethod
    def reset(self) -> None: ...

    def get_current_step(self):
        return self.trajectory.steps[-1] if self.trajectory.steps else None


class ConversationAgentBase(LLMBaseAgent):
    def __init__(self, system_prompt: str = ""):
        self.system_prompt = system_prompt
        self._messages: list = []
        self._trajectory = Trajectory()
        self._pending_obs = None
        self._init_messages(system_prompt)

    def _init_messages(self, system_prompt: str) -> None:
        self._messages = [{"role": "system", "content": system_prompt}] if system_prompt else []

    def _observation_to_messages(self, observation: Any, reward: float, done: bool, info: dict) -> list:
        if observation is None:
            return []
        if isinstance(observation, dict):
            if "question" in observation:
                return [{"role": "user", "content": str(observation["question"])}]
            if "tool_outputs" in observation:
                return [{"role": "tool", "content": str(v), "tool_call_id": k} for k, v in observation["tool_outputs"].items()]
            return [{"role": "user", "content": str(observation)}]
        return [{"role": "user", "content": str(observation)}]

    @property
    def chat_completions(self) -> list:
        return self._messages

    @property
    def trajectory(self) -> Trajectory:
        return self._trajectory

    def update_from_env(self, observation, reward: float = 0.0, done: bool = False, info=None, **kwargs) -> None:
        info = info or {}
        step = self.get_current_step()
        if step is not None:
            step.observation, step.reward, step.done = observation, reward, done
            step.info.update(info)
        self._messages.extend(self._observation_to_messages(observation, reward, done, info))

    def reset(self) -> None:
        self._trajectory = Trajectory()
        self._init_messages(self.system_prompt)
