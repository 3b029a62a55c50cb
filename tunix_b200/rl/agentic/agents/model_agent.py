"""Single-turn agent: the model's response is the action (tunix/rl/agentic/agents/model_agent.py)."""
from __future__ import annotations

import copy

from .agent_types import Action, Step
from .base_agent import ConversationAgentBase


class ModelAgent(ConversationAgentBase):
    def update_from_model(self, response: str, **kwargs) -> Action:
        step = Step(chat_completions=copy.deepcopy(self._messages), model_response=response, action=Action(action=response))
        self._messages.append({"role": "assistant", "content": response})
        self._trajectory.steps.append(step)
        return step.action
