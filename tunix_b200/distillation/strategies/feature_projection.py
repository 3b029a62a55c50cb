"""Feature distillation through learned projections (tunix/distillation/strategies/feature_projection.py).
The projector's parameters are trained together with the student (`extra_trainable_modules`)."""
from __future__ import annotations

import torch

from ..feature_extraction.projection import FeatureProjector
from .base_strategy import task_loss
from .feature_pooling import FeaturePoolingStrategy


class FeatureProjectionStrategy(FeaturePoolingStrategy):
    def __init__(self, student_layers, teacher_layers, student_dim: int, teacher_dim: int, alpha: float = 0.5,
                 dtype=torch.float32, device=None):
        super().__init__(student_layers, teacher_layers, alpha, loss="mse")
        self.projector = FeatureProjector({f"layers.{i}": student_dim for i in student_layers},
                                          {f"layers.{i}": teacher_dim for i in student_layers}, dtype, device)

    @property
    def extra_trainable_modules(self):
        return [self.projector]

    def compute_loss(self, student_output, teacher_output, inputs):
        m = inputs["input_mask"].float()
        tot = 0.0
        for si, ti in zip(self.student_layers, self.teacher_layers):
            s = self.projector(f"layers.{si}", student_output["features"][f"layers.{si}"]).float()
            t = teacher_output["features"][f"layers.{ti}"].float()
            tot = tot + (((s - t) ** 2).mean(-1) * m).sum() / m.sum().clamp(min=1.0)
        tot = tot / max(len(self.student_layers), 1)
        return self.alpha * tot + (1 - self.alpha) * task_loss(student_output["logits"], inputs)
