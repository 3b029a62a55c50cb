"""Short forms of long id lists for log lines (tunix/experimental/common/logging_utils.py:22-46)."""
from __future__ import annotations

from typing import Any, Sequence


def summarize_list(input_list: Sequence[Any], max_length: int = 4) -> str:
    """`[a, b, ..., y, z]`: at most `max_length` entries, the head gets the odd one; empty and None entries are left out."""
    items = [str(x) for x in input_list if x is not None and str(x) != ""]
    if not items:
        return "[]"
    if max_length < 2:
        raise ValueError(f"max_length must be at least 2, got {max_length}")
    if len(items) <= max_length:
        return f"[{', '.join(items)}]"
    tail = max_length // 2
    head = max_length - tail
    return f"[{', '.join(items[:head])}, ..., {', '.join(items[-tail:])}]"


summarize_ids = summarize_list
