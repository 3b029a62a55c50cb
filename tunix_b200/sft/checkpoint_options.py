"""Checkpointing policy objects (tunix/sft/checkpoint_options.py:1-271).

`CheckpointingOptions` (common/configs.py) is the concrete dataclass; this module adds the protocol other
option objects can satisfy, the reference's defaults, and the dict form the CLI accepts."""
from __future__ import annotations

from typing import Any, Optional, Protocol, runtime_checkable

from ..common.configs import CheckpointingOptions

DEFAULT_SAVE_INTERVAL_SECS = 180.0
DEFAULT_MAX_TO_KEEP = 3
DEFAULT_ASYNC_TIMEOUT_SECS = 1200.0


@runtime_checkable
class CheckpointingOptionsLike(Protocol):
    save_interval_steps: Optional[int]
    max_to_keep: Optional[int]


def default_options() -> CheckpointingOptions:
    """Save at most every 180 s, keep the latest 3, asynchronously."""
    return from_dict({})


def from_dict(d: Optional[dict]) -> CheckpointingOptions:
    d = dict(d or {})
    import dataclasses
    names = {f.name for f in dataclasses.fields(CheckpointingOptions)}
    unknown = set(d) - names
    if unknown:
        raise ValueError(f"unknown checkpointing options {sorted(unknown)}; known: {sorted(names)}")
    return CheckpointingOptions(**d)


def resolve(options: Any) -> CheckpointingOptions:
    """None -> defaults; dict -> dataclass; objects with the protocol's attributes are read field by field."""
    if options is None:
        return default_options()
    if isinstance(options, CheckpointingOptions):
        return options
    if isinstance(options, dict):
        return from_dict(options)
    import dataclasses
    return CheckpointingOptions(**{f.name: getattr(options, f.name) for f in dataclasses.fields(CheckpointingOptions)
                                   if hasattr(options, f.name)})
