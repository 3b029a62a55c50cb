"""Logit distillation: a small student learns the next-token distribution of a larger frozen teacher.

    PYTHONPATH=. python examples/distillation/logit_distillation.py [--device cuda] [--steps 60] [--top-k 64]

Random-init models and synthetic tokens keep the example self-contained; with real checkpoints build the two models
with `AutoModel.from_pretrained` instead. The loss is alpha * T^2 * KL(teacher_T || student_T) + (1 - alpha) * CE;
`--top-k` restricts the KL to the teacher's k most likely tokens per position (the rest is one bucket), which is
what makes 128k-entry vocabularies affordable. Other strategies (`AttentionTransferStrategy`,
`FeaturePoolingStrategy`, `FeatureProjectionStrategy`) drop in for `LogitStrategy`."""
import argparse

import torch

from tunix_b200 import optim
from tunix_b200.common.configs import TrainingConfig
from tunix_b200.distillation.distillation_trainer import DistillationTrainer
from tunix_b200.distillation.strategies import LogitStrategy
from tunix_b200.models.config import ModelConfig
from tunix_b200.models.transformer import create_model
from tunix_b200.sft.peft_trainer import TrainingInput


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--temperature", type=float, default=2.0)
    ap.add_argument("--alpha", type=float, default=0.7)
    a = ap.parse_args()
    dev = torch.device(a.device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    teacher_cfg = ModelConfig(family="llama3", num_layers=4, vocab_size=4096, embed_dim=512, hidden_dim=1536, num_heads=8, head_dim=64,
                              num_kv_heads=2, dtype=dtype, max_position=256)
    student_cfg = teacher_cfg.replace(num_layers=2, embed_dim=256, hidden_dim=768, num_heads=4)
    teacher, student = create_model(teacher_cfg, device=dev, seed=0), create_model(student_cfg, device=dev, seed=1)
    g = torch.Generator().manual_seed(0)
    batches = [TrainingInput(torch.randint(0, teacher_cfg.vocab_size, (8, 128), generator=g).to(dev), torch.ones(8, 128, device=dev))
               for _ in range(a.steps)]
    strategy = LogitStrategy(temperature=a.temperature, alpha=a.alpha, teacher_top_k=a.top_k or None)
    cfg = TrainingConfig(eval_every_n_steps=10**9, max_steps=a.steps, pbar_description=None)
    trainer = DistillationTrainer(student, teacher, strategy, optim.AdamW(1e-3, weight_decay=0.0), cfg)
    trainer.train(batches)
    hist = trainer.metrics_logger.get_metric_history("", "loss", "train")
    print(f"distillation loss: first {hist[0]:.4f} -> last {hist[-1]:.4f} over {len(hist)} steps "
          f"(student {student_cfg.num_params() / 1e6:.1f}M, teacher {teacher_cfg.num_params() / 1e6:.1f}M parameters)")


if __name__ == "__main__":
    main()
