"""Tool calls out of whatever an agent's action looks like (tunix/experimental/trajectory/action_converter.py:28-379).

`extract_tool_calls(action)` returns ATIF `ToolCall`s or None. It unwraps `Action`-like objects (an `.action`
attribute), then recognises, in this order:

  objects     `ToolCall`s as they are; dataclasses / objects with `to_dict()` / plain objects through their fields
  dicts       OpenAI `{"id", "type": "function", "function": {"name", "arguments"}}`; Anthropic
              `{"type": "tool_use", "id", "name", "input"}`; flat `{"name" | "tool" | ..., "arguments" | "args" | ...}`
              (without an argument key the remaining keys are the arguments; without a name the call is "action")
  lists       each element as above, ids `call_1`, `call_2`, ... where none is given
  strings     JSON (optionally inside a markdown fence); `<tool_call>` / `<function_call>` blocks holding JSON or
              `<name>` + `<arguments>` tags; `<function=NAME><parameter=KEY>VALUE` and `<invoke name="NAME">` blocks

Numbers, booleans and arrays (discrete or continuous control actions) are not tool calls. Argument strings are parsed
as JSON objects; anything else yields empty arguments rather than an error."""
from __future__ import annotations

import dataclasses
import json
import logging
import re
from typing import Any, List, Optional

import numpy as np

from .trajectory import ToolCall

log = logging.getLogger(__name__)
_ID_KEYS = ("tool_call_id", "call_id", "id")
_NAME_KEYS = ("function_name", "tool_name", "name", "tool", "function")
_ARG_KEYS = ("arguments", "args", "parameters", "params", "input", "inputs")
_META = frozenset(_ID_KEYS + _NAME_KEYS + ("type",))
_NOT_TOOLS = (int, float, bool, np.number, np.ndarray)
_BLOCK = re.compile(r"<(?:tool_call|function_call)>(.*?)(?:</(?:tool_call|function_call)>|$)", re.DOTALL)
_XML_FN = re.compile(r"<(?:function|invoke)(?:\s*=\s*|\s+name=\s*)([^>]+)>(.*?)(?:</(?:function|invoke)>|$)", re.DOTALL)
_XML_PARAM = re.compile(r"<parameter(?:\s*=\s*|\s+name=\s*)([^>]+)>(.*?)(?:</parameter>|$)", re.DOTALL)
_TAG_NAME = re.compile(r"<(?:name|function_name)>(.*?)</(?:name|function_name)>", re.DOTALL)
_TAG_ARGS = re.compile(r"<(arguments|parameters|args|params|input)>(.*?)</\1>", re.DOTALL)


def _first(get, keys):
    for k in keys:
        v = get(k)
        if v is not None:
            return v
    return None


def _strip_fence(s: str) -> str:
    s = s.strip()
    if s.startswith("```"):
        lines = s.splitlines()[1:]
        if lines and lines[-1].strip() == "```":
            lines = lines[:-1]
        s = "\n".join(lines).strip()
    return s


def _as_dict(obj: Any) -> Optional[dict]:
    if isinstance(obj, dict):
        return obj
    if callable(getattr(obj, "to_dict", None)):
        d = obj.to_dict()
        if isinstance(d, dict):
            return d
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        return dataclasses.asdict(obj)
    if hasattr(obj, "__dict__") and not isinstance(obj, type):
        return dict(vars(obj))
    return None


def _arguments(raw: Any) -> dict:
    if raw is None:
        return {}
    d = _as_dict(raw)
    if d is not None:
        return d
    if isinstance(raw, str):
        text = _strip_fence(raw)
        if text:
            try:
                parsed = json.loads(text)
                if isinstance(parsed, dict):
                    return parsed
            except ValueError as e:
                log.warning("tool-call arguments are not JSON: %s", e)
    return {}


def _call(call_id, name, raw_args) -> ToolCall:
    return ToolCall(tool_call_id=str(call_id), function_name=str(name or "action"), arguments=_arguments(raw_args))


def _from_dict(item: dict, default_id: str) -> Optional[ToolCall]:
    call_id = _first(item.get, _ID_KEYS) or default_id
    rest = lambda d: {k: v for k, v in d.items() if k not in _META}         # noqa: E731
    fn = item.get("function")
    if isinstance(fn, dict):                                                  # OpenAI
        args = _first(fn.get, _ARG_KEYS)
        return _call(call_id, _first(fn.get, _NAME_KEYS), rest(fn) if args is None and len(fn) > 1 else args)
    if item.get("type") == "tool_use":                                        # Anthropic
        args = _first(item.get, _ARG_KEYS)
        return _call(call_id, _first(item.get, _NAME_KEYS), rest(item) if args is None and len(item) > 2 else args)
    name, args = _first(item.get, _NAME_KEYS), _first(item.get, _ARG_KEYS)    # flat
    if args is None:
        if name is not None:
            args = rest(item)
        else:
            if item and not {k for k in item if k not in _ID_KEYS and k != "type"}:
                return None                                                   # only an id / a type: nothing is called
            name, args = "action", item
    return _call(call_id, name, args)


def _from_object(item: Any, default_id: str) -> Optional[ToolCall]:
    if item is None or isinstance(item, _NOT_TOOLS):
        return None
    if isinstance(item, ToolCall):
        return item
    d = _as_dict(item)
    if d is not None:
        return _from_dict(d, default_id)
    name = _first(lambda k: getattr(item, k, None), _NAME_KEYS)
    if name is None:
        return None
    return _call(_first(lambda k: getattr(item, k, None), _ID_KEYS) or default_id, name,
                 _first(lambda k: getattr(item, k, None), _ARG_KEYS))


def _from_xml(text: str, start: int = 1) -> Optional[List[ToolCall]]:
    calls = []
    for m in _XML_FN.finditer(text):
        name, body = m.group(1).strip().strip("\"'"), m.group(2).strip()
        if not name:
            continue
        params = _XML_PARAM.findall(body)
        clean = _strip_fence(body)
        if params:
            args: Any = {k.strip().strip("\"'"): v.strip() for k, v in params}
        elif clean.startswith("{"):
            args = clean
        else:
            args = {"input": body} if body else {}
        calls.append(_call(f"call_{start + len(calls)}", name, args))
    return calls or None


def _from_string(text: str) -> Optional[List[ToolCall]]:
    text = text.strip()
    if not text:
        return None
    clean = _strip_fence(text)
    if clean.startswith(("{", "[")):
        try:
            parsed = json.loads(clean)
            calls = _from_payload(parsed) if isinstance(parsed, (dict, list)) else None
            if calls:
                return calls
        except ValueError as e:
            log.warning("action text looks like JSON but is not: %s", e)
    if "<tool_call>" in text or "<function_call>" in text:
        calls: list = []
        for block in _BLOCK.findall(text):
            b = _strip_fence(block.strip())
            if not b:
                continue
            got = None
            if b.startswith(("{", "[")):
                try:
                    parsed = json.loads(b)
                    if isinstance(parsed, dict):
                        one = _from_dict(parsed, f"call_{len(calls) + 1}")
                        got = [one] if one else None
                    elif isinstance(parsed, list):
                        got = _from_payload(parsed)
                except ValueError as e:
                    log.warning("tool-call block is not JSON: %s", e)
            if got is None:
                nm = _TAG_NAME.search(b)
                if nm:
                    am = _TAG_ARGS.search(b)
                    got = [_call(f"call_{len(calls) + 1}", nm.group(1).strip(), am.group(2).strip() if am else "{}")]
            if got is None and ("<function" in b or "<invoke" in b):
                got = _from_xml(b, len(calls) + 1)
            if got:
                calls.extend(got)
        if calls:
            return calls
    if "<function" in text or "<invoke" in text:
        return _from_xml(text)
    return None


def _from_payload(payload: Any) -> Optional[List[ToolCall]]:
    if payload is None or isinstance(payload, _NOT_TOOLS):
        return None
    if isinstance(payload, (dict, list, tuple, str)) and not payload:
        return None
    if isinstance(payload, str):
        return _from_string(payload)
    if isinstance(payload, (list, tuple)):
        calls: list = []
        for item in payload:
            if isinstance(item, str):
                calls.extend(_from_string(item) or [])
            else:
                one = _from_object(item, f"call_{len(calls) + 1}")
                if one:
                    calls.append(one)
        return calls or None
    one = _from_object(payload, "call_1")
    return [one] if one else None


def extract_tool_calls(action: Any) -> Optional[List[ToolCall]]:
    payload = action
    while payload is not None and not isinstance(payload, (ToolCall, dict, str, list, tuple) + _NOT_TOOLS) \
            and hasattr(payload, "action") and not any(hasattr(payload, k) for k in _NAME_KEYS):
        payload = payload.action
    return _from_payload(payload)
