"""Dataset coordinates of prompts (tunix/experimental/common/tagging.py:24-81). The coordinates come from the
position in the dataset alone, so they are the same after a restart and on a retry; a batch-ordered consumer routes
and orders on `batch_idx`."""
from __future__ import annotations

import copy
import dataclasses
import logging
from typing import Any, Mapping

log = logging.getLogger(__name__)


def prompt_coordinates(prompt_idx: int, full_batch_size: int) -> dict:
    return {"prompt_idx": int(prompt_idx), "batch_idx": int(prompt_idx) // full_batch_size,
            "intra_batch_idx": int(prompt_idx) % full_batch_size}


def tag_prompt(prompt_item: Any, coordinates: Mapping[str, int]) -> Any:
    """A copy of the item whose `metadata` carries the coordinates (they win over same-named keys: the dataset position
    is the only authority on them). The item itself is never changed; an object whose metadata cannot be replaced is
    returned as it is, with a warning."""
    if isinstance(prompt_item, Mapping):
        out = dict(prompt_item)
        out["metadata"] = {**(out.get("metadata") or {}), **coordinates}
        return out
    metadata = {**(getattr(prompt_item, "metadata", None) or {}), **coordinates}
    if dataclasses.is_dataclass(prompt_item) and any(f.name == "metadata" for f in dataclasses.fields(prompt_item)):
        return dataclasses.replace(prompt_item, metadata=metadata)          # also works for frozen dataclasses
    out = copy.copy(prompt_item)
    try:
        out.metadata = metadata
    except (AttributeError, TypeError):
        log.warning("cannot tag prompt coordinates onto a %s: batch-ordered consumption needs a `metadata` mapping on every "
                    "prompt item", type(prompt_item).__name__)
        return prompt_item
    return out
