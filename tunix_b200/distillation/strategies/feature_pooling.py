"""Feature distillation with pooling to a common width (tunix/distillation/strategies/feature_pooling.py)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..feature_extraction.pooling import avg_pool_to
from ..feature_extraction.sowed_module import pop_sowed_intermediates, sow_intermediates
from .base_strategy import BaseStrategy, task_loss


def _forward_with_features(model, inputs, layers):
    names = {f"layers.{i}" for i in layers}
    with sow_intermediates(model, lambda n, m: n in names) as store:
        logits, _ = model(inputs["input_tokens"], positions=inputs.get("positions"), segment_ids=inputs.get("segment_ids"))
        feats = pop_sowed_intermediates(store)
    return {"logits": logits, "features": feats}


class FeaturePoolingStrategy(BaseStrategy):
    def __init__(self, student_layers, teacher_layers, alpha: float = 0.5, loss: str = "cosine"):
        assert len(student_layers) == len(teacher_layers)
        self.student_layers, self.teacher_layers, self.alpha, self.loss = list(student_layers), list(teacher_layers), alpha, loss

    def student_forward(self, model, inputs):
        return _forward_with_features(model, inputs, self.student_layers)

    @torch.no_grad()
    def get_teacher_outputs(self, teacher, inputs):
        return _forward_with_features(teacher, inputs, self.teacher_layers)

    def _pair_loss(self, s, t, mask):
        d = min(s.shape[-1], t.shape[-1])
        s, t = avg_pool_to(s.float(), d), avg_pool_to(t.float(), d)
        per_tok = 1.0 - F.cosine_similarity(s, t, dim=-1) if self.loss == "cosine" else ((s - t) ** 2).mean(-1)
        return (per_tok * mask).sum() / mask.sum().clamp(min=1.0)

    def compute_loss(self, student_output, teacher_output, inputs):
        m = inputs["input_mask"].float()
        tot = 0.0
        for si, ti in zip(self.student_layers, self.teacher_layers):
            tot = tot + self._pair_loss(student_output["features"][f"layers.{si}"], teacher_output["features"][f"layers.{ti}"], m)
        tot = tot / max(len(self.student_layers), 1)
        return self.alpha * tot + (1 - self.alpha) * task_loss(student_output["logits"], inputs)
