"""Diffusion-LM supervised fine-tuning on PeftTrainer (tunix/sft/diffusion.py:31-93): weighted cross-entropy on
target-aligned logits, no one-token shift; which positions count is the batch adapter's business."""
from __future__ import annotations

import torch

from ..diffusion import interfaces, types
from .utils import LossOutput, WeightedMetric


def diffusion_loss_fn(model, batch: types.DiffusionTokenBatch, logits_fn: interfaces.DiffusionLogitsFn) -> LossOutput:
    logits = interfaces.compute_diffusion_logits(model, batch, logits_fn).float()
    weights = torch.as_tensor(batch.loss_weights, device=logits.device).float()
    targets = torch.as_tensor(batch.target_ids, device=logits.device).long()
    active = weights > 0
    targets = torch.where(active, targets, torch.zeros_like(targets))
    logp = torch.log_softmax(logits, -1).gather(-1, targets[..., None]).squeeze(-1)
    loss_sum = -(torch.where(active, logp, torch.zeros_like(logp)) * weights).sum()
    return LossOutput(WeightedMetric(loss_sum, weights.sum()))


def configure_diffusion_sft(trainer, batch_adapter: interfaces.DiffusionBatchAdapter, logits_fn: interfaces.DiffusionLogitsFn):
    trainer.with_gen_model_input_fn(lambda raw: {"batch": batch_adapter(raw)})
    trainer.with_loss_fn(lambda model, batch: diffusion_loss_fn(model, batch, logits_fn))
    return trainer
