"""Multi-turn tool environment: executes tool calls, feeds `{"tool_outputs": ...}` back, ends on `finish`
(tunix/rl/agentic/environments/tool_environment.py)."""
from __future__ import annotations

from typing import Any, Callable, Optional

from ..rewards.reward import get_reward_fn
from ..tools.tool_manager import ToolManager
from .base_environment import BaseTaskEnv


class ToolEnvironment(BaseTaskEnv):
    def __init__(self, task: Any = None, tools=None, reward_fn: Optional[Callable] = None, max_steps: int = 10, **kwargs):
        super().__init__(task, max_steps, **kwargs)
        self.tool_manager = tools if isinstance(tools, ToolManager) else ToolManager(tools or {})
        self.reward_fn = get_reward_fn(reward_fn) if isinstance(reward_fn, str) else (reward_fn or get_reward_fn("zero"))

    def _initial_observation(self):
        return self.task if isinstance(self.task, dict) else {"question": self.task}

    def _step_impl(self, action):
        calls = action if isinstance(action, list) else [{"id": "0", "name": "finish", "arguments": {"response": action}}]
        finish = next((c for c in calls if c.get("name") == "finish"), None)
        if finish is not None or self.step_count >= self.max_steps:
            answer = (finish or {}).get("arguments", {}).get("response", "")
            out = self.reward_fn(task=self.task, action=answer)
            return {}, float(out.reward), True, {"response": answer, "metadata": out.metadata}
        outputs = self.tool_manager.execute_calls(calls)
        return {"tool_outputs": {k: str(v) for k, v in outputs.items()}}, 0.0, False, {}
