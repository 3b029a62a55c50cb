"""Distillation strategies on tiny CPU models."""
import pytest
import torch

from tunix_b200 import optim
from tunix_b200.common.configs import TrainingConfig
from tunix_b200.distillation.distillation_trainer import DistillationTrainer
from tunix_b200.distillation.strategies import (AttentionTransferStrategy, FeaturePoolingStrategy,
                                                FeatureProjectionStrategy, LogitStrategy)
from tunix_b200.models.config import ModelConfig
from tunix_b200.models.transformer import create_model
from tunix_b200.sft.peft_trainer import TrainingInput


def _models():
    t = ModelConfig.tiny_llama().replace(num_layers=2, vocab_size=64, embed_dim=48, hidden_dim=96, num_heads=2, head_dim=24,
                                         num_kv_heads=1)
    s = t.replace(num_layers=1, embed_dim=32, hidden_dim=64, head_dim=16)
    return create_model(s, seed=1), create_model(t, seed=0)


def _batch():
    g = torch.Generator().manual_seed(0)
    return TrainingInput(torch.randint(0, 64, (4, 12), generator=g), torch.ones(4, 12))


@pytest.mark.parametrize("make", [
    lambda: LogitStrategy(temperature=2.0, alpha=0.7),
    lambda: LogitStrategy(temperature=1.0, alpha=1.0, teacher_top_k=8),
    lambda: AttentionTransferStrategy([0], [1]),
    lambda: FeaturePoolingStrategy([0], [1]),
    lambda: FeatureProjectionStrategy([0], [1], student_dim=32, teacher_dim=48),
])
def test_strategy_trains_student_only(make):
    student, teacher = _models()
    t_before = [p.detach().clone() for p in teacher.parameters()]
    tc = TrainingConfig(eval_every_n_steps=100, max_steps=6, pbar_description=None)
    tr = DistillationTrainer(student, teacher, make(), optim.AdamW(3e-3, weight_decay=0.0), tc)
    tr.train([_batch()] * 6)
    hist = tr.metrics_logger.get_metric_history("", "loss", "train")
    assert hist[-1] < hist[0]
    for p, q in zip(teacher.parameters(), t_before):
        assert torch.equal(p, q)


def test_logit_kd_is_zero_for_identical_models():
    s, _ = _models()
    strat = LogitStrategy(temperature=2.0, alpha=1.0)
    b = _batch()
    inputs = {"input_tokens": b.input_tokens, "input_mask": b.input_mask}
    out = strat.student_forward(s, inputs)
    assert abs(strat.compute_loss(out, out.detach(), inputs).item()) < 1e-6
