"""Protocols between a diffusion-LM model and the trainer (tunix/diffusion/interfaces.py:25-70)."""
from __future__ import annotations

from typing import Any, Protocol, TypeVar

from .types import DiffusionTokenBatch, validate_diffusion_logits

RawBatchT_contra = TypeVar("RawBatchT_contra", contravariant=True)


class DiffusionBatchAdapter(Protocol[RawBatchT_contra]):
    """Turns whatever the data pipeline yields into a `DiffusionTokenBatch` (noising schedule, masking, weights)."""

    def __call__(self, raw_batch: RawBatchT_contra) -> DiffusionTokenBatch: ...


class DiffusionLogitsFn(Protocol):
    """Scores a batch: logits [batch, length, vocab] whose first two dimensions align with `target_ids`."""

    def __call__(self, model: Any, model_inputs: Any) -> Any: ...


def compute_diffusion_logits(model, batch: DiffusionTokenBatch, logits_fn: DiffusionLogitsFn):
    return validate_diffusion_logits(logits_fn(model, batch.model_inputs), batch)
