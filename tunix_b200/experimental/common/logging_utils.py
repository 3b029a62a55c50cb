"""Short forms of long id lists for log lines (tunix/experimental/common/logging_utils.py:22-46)."""
from __future__ import annotations

from typing import Any, Iterable

_ELLIPSIS = "..."


def _printable(values: Iterable[Any]) -> list:
    """Entries as text; `None` and empty entries carry no information in a log line and are left out."""
    texts = (str(v) for v in values if v is not None)
    return [t for t in texts if t]


def summarize_list(input_list: Iterable[Any], max_length: int = 4) -> str:
    """`[a, b, ..., y, z]`: a list printed whole when it has at most `max_length` printable entries, otherwise its first
    ceil(max_length / 2) and last floor(max_length / 2) entries around an ellipsis."""
    shown = _printable(input_list)
    if shown and max_length < 2:
        raise ValueError(f"max_length must be at least 2, got {max_length}")
    if len(shown) > max_length:
        back = max_length >> 1
        shown = shown[:max_length - back] + [_ELLIPSIS] + shown[len(shown) - back:]
    return "[" + ", ".join(shown) + "]"


summarize_ids = summarize_list
