"""Tool interface with JSON-schema description (tunix/rl/agentic/tools/base_tool.py)."""
from __future__ import annotations

import abc
import asyncio
import dataclasses
from typing import Any, Optional


@dataclasses.dataclass
class ToolOutput:
    name: str
    output: Any = None
    error: Optional[str] = None

    def __str__(self) -> str:
        return f"Error: {self.error}" if self.error else str(self.output)


class BaseTool(abc.ABC):
    name: str = ""
    description: str = ""

    @abc.abstractmethod
    def get_json_schema(self) -> dict: ...

    def apply(self, **kwargs) -> ToolOutput:
        raise NotImplementedError

    async def apply_async(self, **kwargs) -> ToolOutput:
        return await asyncio.get_running_loop().run_in_executor(None, lambda: self.apply(**kwargs))

    def to_mcp_schema(self) -> dict:
        s = self.get_json_schema()["function"]
        return {"name": s["name"], "description": s.get("description", ""), "inputSchema": s.get("parameters", {})}
