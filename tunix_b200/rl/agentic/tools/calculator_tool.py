"""Safe arithmetic calculator tool (tunix/rl/agentic/tools/calculator_tool.py)."""
from __future__ import annotations

import ast
import operator

from .base_tool import BaseTool, ToolOutput

_OPS = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.Div: operator.truediv,
        ast.Pow: operator.pow, ast.Mod: operator.mod, ast.FloorDiv: operator.floordiv, ast.USub: operator.neg,
        ast.UAdd: operator.pos}


def _eval(node):
    if isinstance(node, ast.Constant) and isinstance(node.value, (int, float)):
        return node.value
    if isinstance(node, ast.BinOp) and type(node.op) in _OPS:
        l, r = _eval(node.left), _eval(node.right)
        if isinstance(node.op, ast.Pow) and abs(r) > 64:
            raise ValueError("exponent too large")
        return _OPS[type(node.op)](l, r)
    if isinstance(node, ast.UnaryOp) and type(node.op) in _OPS:
        return _OPS[type(node.op)](_eval(node.operand))
    raise ValueError("unsupported expression")


class CalculatorTool(BaseTool):
    name = "calculator"
    description = "Evaluate an arithmetic expression with + - * / ** % //."

    def get_json_schema(self) -> dict:
        return {"type": "function", "function": {"name": self.name, "description": self.description, "parameters": {
            "type": "object", "properties": {"expression": {"type": "string"}}, "required": ["expression"]}}}

    def apply(self, expression: str = "", **kwargs) -> ToolOutput:
        try:
            return ToolOutput(self.name, output=_eval(ast.parse(expression, mode="eval").body))
        except Exception as e:
            return ToolOutput(self.name, error=f"{type(e).__name__}: {e}")
