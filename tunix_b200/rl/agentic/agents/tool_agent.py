"""Tool-calling agent: parses tool calls out of the model response (tunix/rl/agentic/agents/tool_agent.py)."""
from __future__ import annotations

import copy
import json
import uuid
from typing import Optional

from ..parser.tool_parser import QwenToolParser, ToolParser
from ..tools.base_tool import BaseTool
from .agent_types import Action, Step
from .base_agent import ConversationAgentBase

DEFAULT_TOOL_PROMPT = ("You can call tools. To call one, answer with <tool_call>{\"name\": ..., \"arguments\": {...}}"
                       "</tool_call>. When you are done call the `finish` tool with your final answer.")


class ToolAgent(ConversationAgentBase):
    def __init__(self, system_prompt: str = "", tool_parser: Optional[ToolParser] = None, tools: Optional[dict] = None):
        self.tool_parser = tool_parser or QwenToolParser()
        self.tools: dict = tools or {}
        schemas = [t.get_json_schema() for t in self.tools.values() if isinstance(t, BaseTool)]
        prompt = system_prompt or DEFAULT_TOOL_PROMPT
        if schemas:
            prompt += "\n# Tools\n" + "\n".join(json.dumps(s) for s in schemas)
        super().__init__(prompt)

    def update_from_model(self, response: str, **kwargs) -> Action:
        calls = self.tool_parser.parse(response)
        if not calls:
            calls = [{"name": "finish", "arguments": {"response": response}}]
        for c in calls:
            c.setdefault("id", uuid.uuid4().hex[:8])
        step = Step(chat_completions=copy.deepcopy(self._messages), model_response=response, action=Action(action=calls))
        self._messages.append({"role": "assistant", "content": response})
        self._trajectory.steps.append(step)
        return step.action
