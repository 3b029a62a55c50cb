"""Batch contract of diffusion-LM training (tunix/diffusion/types.py:56-190).

A diffusion language model scores every target position at once, so the batch names, position by position,
the token to predict and how much that position counts; there is no autoregressive shift."""
from __future__ import annotations

import dataclasses
from typing import Any

import numpy as np
import torch


def _leaves(tree) -> list:
    if isinstance(tree, dict):
        return [l for v in tree.values() for l in _leaves(v)]
    if isinstance(tree, (list, tuple)):
        return [l for v in tree for l in _leaves(v)]
    return [] if tree is None else [tree]


def _shape_dtype(name: str, v):
    if isinstance(v, (torch.Tensor, np.ndarray)):
        return tuple(v.shape), v.dtype
    raise TypeError(f"{name} must be a tensor or ndarray, got {type(v).__name__}")


def _is_real(dt) -> bool:
    if isinstance(dt, torch.dtype):
        return dt == torch.bool or dt.is_floating_point or dt in (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)
    return np.issubdtype(dt, np.bool_) or np.issubdtype(dt, np.integer) or np.issubdtype(dt, np.floating)


def _is_int(dt) -> bool:
    if isinstance(dt, torch.dtype):
        return dt in (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)
    return np.issubdtype(dt, np.integer)


@dataclasses.dataclass
class DiffusionTokenBatch:
    model_inputs: Any            # batch-major tensors consumed by the logits callable
    target_ids: Any              # [batch, length] integers
    loss_weights: Any            # [batch, length] nonnegative, finite

    @classmethod
    def create(cls, *, model_inputs, target_ids, loss_weights) -> "DiffusionTokenBatch":
        return cls(model_inputs, target_ids, loss_weights).validate()

    def validate(self) -> "DiffusionTokenBatch":
        tshape, tdt = _shape_dtype("target_ids", self.target_ids)
        if len(tshape) != 2:
            raise ValueError(f"target_ids must have shape [batch, length]; received {tshape}")
        if not _is_int(tdt):
            raise TypeError(f"target_ids must have an integer dtype; received {tdt}")
        wshape, wdt = _shape_dtype("loss_weights", self.loss_weights)
        if wshape != tshape:
            raise ValueError(f"loss_weights must match target_ids shape; received {wshape} and {tshape}")
        if not _is_real(wdt):
            raise TypeError(f"loss_weights must have a real numeric or boolean dtype; received {wdt}")
        w = torch.as_tensor(self.loss_weights).float()
        if not torch.isfinite(w).all():
            raise ValueError("loss_weights must contain only finite values")
        if (w < 0).any():
            raise ValueError("loss_weights must be nonnegative")
        t = torch.as_tensor(self.target_ids)
        if (t[w.to(t.device) > 0] < 0).any():
            raise ValueError("active target_ids must be nonnegative")
        leaves = _leaves(self.model_inputs)
        if not leaves:
            raise ValueError("model_inputs must contain at least one array")
        for i, leaf in enumerate(leaves):
            shape, dt = _shape_dtype(f"model_inputs leaf {i}", leaf)
            if not shape:
                raise ValueError(f"model_inputs leaf {i} must be batch-major, not scalar")
            if shape[0] != tshape[0]:
                raise ValueError(f"model_inputs leaf {i} has batch size {shape[0]}; expected {tshape[0]}")
            if not _is_real(dt):
                raise TypeError(f"model_inputs leaf {i} must have a real numeric or boolean dtype; received {dt}")
        return self


def validate_diffusion_logits(logits, batch: DiffusionTokenBatch):
    shape = tuple(logits.shape)
    want = tuple(batch.target_ids.shape)
    if len(shape) != 3 or shape[:2] != want:
        raise ValueError(f"logits must have shape [batch, length, vocab] aligned with target_ids {want}; received {shape}")
    return logits
