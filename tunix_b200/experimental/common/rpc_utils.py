"""Checks on payloads that cross process boundaries (tunix/experimental/common/rpc_utils.py:21-49)."""
from __future__ import annotations

import dataclasses
from typing import Any, Iterator

import numpy as np

_CONTAINERS = (list, tuple, set, frozenset)


def _children(node: Any) -> Iterator[Any]:
    """What a payload node holds: fields of a dataclass instance, keys and values of a dict, items of a sequence or set."""
    if isinstance(node, dict):
        yield from node
        yield from node.values()
    elif isinstance(node, _CONTAINERS):
        yield from node
    elif dataclasses.is_dataclass(node) and not isinstance(node, type):
        for field in dataclasses.fields(node):
            yield getattr(node, field.name)


def _is_foreign_array(node: Any) -> bool:
    """Array-like (has a shape and a dtype) without being a numpy array: a device tensor, most likely."""
    return not isinstance(node, np.ndarray) and hasattr(node, "dtype") and hasattr(node, "shape")


def validate_wire_safe(obj: object) -> None:
    """Raise TypeError when the payload holds an array that is not a `numpy.ndarray`: a device tensor cannot be
    rebuilt in a process that does not own its memory (and pickling one copies it through the host behind the caller's
    back). Shared objects are visited once, so cyclic payloads terminate."""
    seen: set = set()
    frontier = [obj]
    while frontier:
        node = frontier.pop()
        if id(node) in seen:
            continue
        seen.add(id(node))
        if _is_foreign_array(node):
            kind = type(node)
            raise TypeError(f"wire payload contains a non-numpy array of type {kind.__module__}.{kind.__qualname__}; "
                            "convert device tensors to numpy before serialization")
        if not isinstance(node, np.ndarray):
            frontier.extend(_children(node))
