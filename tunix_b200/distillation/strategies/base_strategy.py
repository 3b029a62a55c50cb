"""Distillation strategy interface (tunix/distillation/strategies/base_strategy.py)."""
from __future__ import annotations

import abc
from typing import Any

import torch


class BaseStrategy(abc.ABC):
    """A strategy defines what is extracted from teacher and student and how the two are compared."""

    def student_forward(self, model, inputs: dict) -> Any:
        logits, _ = model(inputs["input_tokens"], positions=inputs.get("positions"), segment_ids=inputs.get("segment_ids"))
        return logits

    @torch.no_grad()
    def get_teacher_outputs(self, teacher, inputs: dict) -> Any:
        return self.student_forward(teacher, inputs)

    @abc.abstractmethod
    def compute_loss(self, student_output: Any, teacher_output: Any, inputs: dict) -> torch.Tensor: ...

    def compute_eval_loss(self, student_output: Any, inputs: dict) -> torch.Tensor:
        return task_loss(student_output if isinstance(student_output, torch.Tensor) else student_output["logits"], inputs)

    def get_train_loss(self, student, teacher_output, inputs: dict) -> torch.Tensor:
        return self.compute_loss(self.student_forward(student, inputs), teacher_output, inputs)

    def get_eval_loss(self, student, inputs: dict) -> torch.Tensor:
        return self.compute_eval_loss(self.student_forward(student, inputs), inputs)


def task_loss(logits: torch.Tensor, inputs: dict) -> torch.Tensor:
    """Masked next-token cross entropy."""
    toks, mask = inputs["input_tokens"], inputs["input_mask"]
    lsm = torch.log_softmax(logits[:, :-1].float(), -1)
    nll = -lsm.gather(-1, toks[:, 1:].long().unsqueeze(-1)).squeeze(-1)
    m = mask[:, 1:].float()
    return (nll * m).sum() / m.sum().clamp(min=1.0)
