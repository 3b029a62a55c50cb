"""Checks on payloads that cross process boundaries (tunix/experimental/common/rpc_utils.py:21-49)."""
from __future__ import annotations

import dataclasses

import numpy as np


def validate_wire_safe(obj: object) -> None:
    """Raise TypeError when the payload holds an array that is not a `numpy.ndarray`: a device tensor cannot be
    rebuilt in a process that does not own its memory (and pickling one copies it through the host behind the caller's
    back). Walks dataclasses, dicts (keys and values), lists, tuples and sets; shared objects are visited once."""
    stack, seen = [obj], set()
    while stack:
        v = stack.pop()
        if id(v) in seen:
            continue
        seen.add(id(v))
        if isinstance(v, np.ndarray):
            continue
        if dataclasses.is_dataclass(v) and not isinstance(v, type):
            stack.extend(getattr(v, f.name) for f in dataclasses.fields(v))
        elif isinstance(v, dict):
            stack.extend(v.keys())
            stack.extend(v.values())
        elif isinstance(v, (list, tuple, set, frozenset)):
            stack.extend(v)
        elif hasattr(v, "shape") and hasattr(v, "dtype"):
            raise TypeError(f"wire payload contains a non-numpy array of type {type(v).__module__}.{type(v).__qualname__}; "
                            "convert device tensors to numpy before serialization")
