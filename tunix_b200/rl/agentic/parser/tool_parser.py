"""Tool-call parsers (tunix/rl/agentic/parser/tool_parser/*): Qwen `<tool_call>{json}</tool_call>` and
Gemini-style ```tool_code / function-call JSON blocks."""
from __future__ import annotations

import abc
import json
import re


class ToolParser(abc.ABC):
    @abc.abstractmethod
    def parse(self, response: str) -> list: ...

    @abc.abstractmethod
    def get_tool_prompt(self, schemas: list) -> str: ...


class QwenToolParser(ToolParser):
    _RE = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)

    def parse(self, response: str) -> list:
        out = []
        for m in self._RE.finditer(response):
            try:
                d = json.loads(m.group(1))
            except json.JSONDecodeError:
                continue
            if "name" in d:
                out.append({"name": d["name"], "arguments": d.get("arguments", d.get("parameters", {})) or {}})
        return out

    def get_tool_prompt(self, schemas: list) -> str:
        return ("# Tools\nYou may call one or more functions. Signatures:\n<tools>\n" + "\n".join(json.dumps(s) for s in schemas)
                + "\n</tools>\nReturn each call as <tool_call>{\"name\": <name>, \"arguments\": <args>}</tool_call>")


class GeminiToolParser(ToolParser):
    _RE = re.compile(r"```(?:tool_code|json)?\s*(\{.*?\})\s*```", re.S)

    def parse(self, response: str) -> list:
        out = []
        for m in self._RE.finditer(response):
            try:
                d = json.loads(m.group(1))
            except json.JSONDecodeError:
                continue
            fc = d.get("functionCall", d.get("function_call", d))
            if "name" in fc:
                out.append({"name": fc["name"], "arguments": fc.get("args", fc.get("arguments", {})) or {}})
        return out

    def get_tool_prompt(self, schemas: list) -> str:
        return "Available functions:\n" + "\n".join(json.dumps(s) for s in schemas) + \
               "\nCall a function with ```tool_code\n{\"name\": ..., \"args\": {...}}\n```"
