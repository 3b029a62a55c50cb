"""Tool registry and parallel execution of tool calls (tunix/rl/agentic/tools/tool_manager.py)."""
from __future__ import annotations

import asyncio
import concurrent.futures as cf
from typing import Iterable

from .base_tool import BaseTool, ToolOutput


class ToolManager:
    def __init__(self, tools: Iterable[BaseTool] | dict):
        self.tools = dict(tools) if isinstance(tools, dict) else {t.name: t for t in tools}

    def get_schemas(self) -> list:
        return [t.get_json_schema() for t in self.tools.values()]

    def run(self, name: str, **arguments) -> ToolOutput:
        if name not in self.tools:
            return ToolOutput(name, error=f"unknown tool {name!r}")
        try:
            return self.tools[name].apply(**arguments)
        except Exception as e:
            return ToolOutput(name, error=f"{type(e).__name__}: {e}")

    def execute_calls(self, calls: list, parallel: bool = True) -> dict:
        """calls: [{id, name, arguments}] -> {id: ToolOutput}."""
        if not parallel or len(calls) <= 1:
            return {c["id"]: self.run(c["name"], **(c.get("arguments") or {})) for c in calls}
        with cf.ThreadPoolExecutor(max_workers=len(calls)) as ex:
            futs = {c["id"]: ex.submit(self.run, c["name"], **(c.get("arguments") or {})) for c in calls}
            return {k: f.result() for k, f in futs.items()}

    async def execute_calls_async(self, calls: list) -> dict:
        async def one(c):
            t = self.tools.get(c["name"])
            if t is None:
                return c["id"], ToolOutput(c["name"], error=f"unknown tool {c['name']!r}")
            try:
                return c["id"], await t.apply_async(**(c.get("arguments") or {}))
            except Exception as e:
                return c["id"], ToolOutput(c["name"], error=f"{type(e).__name__}: {e}")
        return dict(await asyncio.gather(*(one(c) for c in calls)))
