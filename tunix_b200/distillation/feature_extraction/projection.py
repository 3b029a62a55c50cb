"""Learned linear projections from student to teacher feature width
(tunix/distillation/feature_extraction/projection.py)."""
from __future__ import annotations

import torch
import torch.nn as nn


class FeatureProjector(nn.Module):
    def __init__(self, student_dims: dict, teacher_dim_of: dict, dtype=torch.float32, device=None):
        super().__init__()
        self.proj = nn.ModuleDict({k.replace(".", "__"): nn.Linear(d, teacher_dim_of[k], bias=False, dtype=dtype, device=device)
                                   for k, d in student_dims.items()})

    def forward(self, name: str, x: torch.Tensor) -> torch.Tensor:
        return self.proj[name.replace(".", "__")](x.to(self.proj[name.replace(".", "__")].weight.dtype))
