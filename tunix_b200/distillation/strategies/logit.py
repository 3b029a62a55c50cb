"""Logit distillation: alpha * T^2 * KL(teacher_T || student_T) + (1 - alpha) * CE, optional teacher top-k
(tunix/distillation/strategies/logit.py:95-169)."""
from __future__ import annotations

from typing import Optional

import torch

from .base_strategy import BaseStrategy, task_loss


class LogitStrategy(BaseStrategy):
    def __init__(self, temperature: float = 2.0, alpha: float = 0.5, teacher_top_k: Optional[int] = None):
        if temperature <= 0:
            raise ValueError("temperature must be positive")
        if not 0.0 <= alpha <= 1.0:
            raise ValueError("alpha must be in [0, 1]")
        self.temperature, self.alpha, self.teacher_top_k = temperature, alpha, teacher_top_k

    def compute_loss(self, student_output, teacher_output, inputs):
        T = self.temperature
        s, t = student_output.float() / T, teacher_output.float() / T
        if self.teacher_top_k:
            kth = torch.topk(t, self.teacher_top_k, dim=-1).values[..., -1:]
            keep = t >= kth
            t = t.masked_fill(~keep, -float("inf"))
            s = s.masked_fill(~keep, -float("inf"))
        tp = torch.softmax(t, -1)
        kl = (tp * (torch.log_softmax(t, -1) - torch.log_softmax(s, -1))).nan_to_num(0.0).sum(-1)
        m = inputs["input_mask"].float()
        distill = (kl * m).sum() / m.sum().clamp(min=1.0) * T * T
        return self.alpha * distill + (1.0 - self.alpha) * task_loss(student_output, inputs)
