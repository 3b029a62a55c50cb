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
    batch, within = divmod(int(prompt_idx), int(full_batch_size))
    return {"prompt_idx": int(prompt_idx), "batch_idx": batch, "intra_batch_idx": within}


def _with_metadata(item: Any, metadata: dict) -> Any:
    """`item` with its `metadata` replaced, by whatever means its type allows; raises when there is none."""
    if isinstance(item, Mapping):
        return {**item, "metadata": metadata}
    if dataclasses.is_dataclass(item) and not isinstance(item, type) and "metadata" in {f.name for f in dataclasses.fields(item)}:
        return dataclasses.replace(item, metadata=metadata)          # works for frozen dataclasses too
    clone = copy.copy(item)
    clone.metadata = metadata                                        # AttributeError / TypeError for slots, ints, ...
    return clone


def tag_prompt(prompt_item: Any, coordinates: Mapping[str, int]) -> Any:
    """A copy of the item whose `metadata` carries the coordinates (they win over same-named keys: the dataset position
    is the only authority on them). The item itself is never changed; an object whose metadata cannot be replaced is
    returned as it is, with a warning."""
    old = prompt_item.get("metadata") if isinstance(prompt_item, Mapping) else getattr(prompt_item, "metadata", None)
    merged = dict(old or {})
    merged.update(coordinates)
    try:
        return _with_metadata(prompt_item, merged)
    except (AttributeError, TypeError):
        log.warning("cannot tag prompt coordinates onto a %s: batch-ordered consumption needs a `metadata` mapping on every "
                    "prompt item", type(prompt_item).__name__)
        return prompt_item
