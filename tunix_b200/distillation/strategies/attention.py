"""Attention transfer: match head-averaged attention maps of selected layers
(tunix/distillation/strategies/attention.py)."""
from __future__ import annotations

import math

import torch

from ...models.transformer import Attention
from ..feature_extraction.sowed_module import pop_sowed_intermediates, sow_intermediates
from .base_strategy import BaseStrategy, task_loss


def _attention_maps(model, inputs, layer_filter):
    """Run the model and rebuild softmax(QK^T) (averaged over heads) for every matched attention module."""
    maps = {}
    handles = []
    for name, mod in model.named_modules():
        if isinstance(mod, Attention) and layer_filter(name):
            def pre(m, args, kwargs, _name=name):
                x = args[0]
                B, T, _ = x.shape
                cfg = m.cfg
                q = m.q_proj(x).view(B, T, cfg.num_heads, cfg.head_dim).float()
                k = m.k_proj(x).view(B, T, cfg.num_kv_heads, cfg.head_dim).float()
                k = k.repeat_interleave(cfg.num_heads // cfg.num_kv_heads, dim=2)
                s = torch.einsum("bqnh,bknh->bnqk", q, k) * m.scale
                causal = torch.tril(torch.ones(T, T, dtype=torch.bool, device=x.device))
                maps[_name] = torch.softmax(s.masked_fill(~causal, -float("inf")), -1).mean(1)
            handles.append(mod.register_forward_pre_hook(pre, with_kwargs=True))
    try:
        logits, _ = model(inputs["input_tokens"], positions=inputs.get("positions"), segment_ids=inputs.get("segment_ids"))
    finally:
        for h in handles:
            h.remove()
    return {"logits": logits, "maps": maps}


class AttentionTransferStrategy(BaseStrategy):
    def __init__(self, student_layers, teacher_layers, alpha: float = 0.5):
        assert len(student_layers) == len(teacher_layers)
        self.student_layers, self.teacher_layers, self.alpha = list(student_layers), list(teacher_layers), alpha

    def student_forward(self, model, inputs):
        names = {f"layers.{i}.self_attn" for i in self.student_layers}
        return _attention_maps(model, inputs, lambda n: n in names)

    @torch.no_grad()
    def get_teacher_outputs(self, teacher, inputs):
        names = {f"layers.{i}.self_attn" for i in self.teacher_layers}
        return _attention_maps(teacher, inputs, lambda n: n in names)

    def compute_loss(self, student_output, teacher_output, inputs):
        loss = 0.0
        for si, ti in zip(self.student_layers, self.teacher_layers):
            sm = student_output["maps"][f"layers.{si}.self_attn"]
            tm = teacher_output["maps"][f"layers.{ti}.self_attn"]
            loss = loss + ((sm - tm) ** 2).mean()
        loss = loss / max(len(self.student_layers), 1)
        return self.alpha * loss + (1 - self.alpha) * task_loss(student_output["logits"], inputs)
