"""DistillationTrainer: PeftTrainer whose `_prepare_inputs` runs the frozen teacher and whose loss is defined
by a strategy (tunix/distillation/distillation_trainer.py:41-170)."""
from __future__ import annotations

import dataclasses
from typing import Any

import torch

from ..common.configs import TrainingConfig
from ..sft.peft_trainer import PeftTrainer, TrainingInput
from .strategies.base_strategy import BaseStrategy


@dataclasses.dataclass
class DistillationInput:
    inputs: dict
    teacher_output: Any


class DistillationTrainer(PeftTrainer):
    def __init__(self, student_model, teacher_model, strategy: BaseStrategy, optimizer, training_config: TrainingConfig,
                 metrics_logger=None):
        for m in getattr(strategy, "extra_trainable_modules", []):
            student_model.add_module("_distill_" + type(m).__name__.lower(), m)
        super().__init__(student_model, optimizer, training_config, metrics_logger)
        self.teacher_model = teacher_model
        self.strategy = strategy
        for p in teacher_model.parameters():
            p.requires_grad_(False)
        self.loss_fn = lambda model, batch: strategy.get_train_loss(model, batch.teacher_output, batch.inputs)
        self.eval_loss_fn = lambda model, batch: strategy.get_eval_loss(model, batch.inputs)
        self.gen_model_input_fn = lambda b: {"batch": b}

    def _shard_and_move(self, batch):
        return batch

    @torch.no_grad()
    def _prepare_inputs(self, batch: Any) -> DistillationInput:
        from ..sft import sharding_utils
        from ..sft.peft_trainer import _to_device
        batch = sharding_utils.shard_input(batch, self.config.data_sharding_axis)
        if isinstance(batch, TrainingInput):
            inputs = {"input_tokens": batch.input_tokens, "input_mask": batch.input_mask}
        else:
            inputs = dict(batch)
        inputs = {k: _to_device(v, self.device) for k, v in inputs.items()}
        was = self.teacher_model.training
        self.teacher_model.eval()
        teacher_out = self.strategy.get_teacher_outputs(self.teacher_model, inputs)
        self.teacher_model.train(was)
        return DistillationInput(inputs, teacher_out)
