"""DPO / ORPO trainer on CPU."""
import math

import numpy as np
import torch

from tunix_b200 import optim
from tunix_b200.lora import LoraProvider, apply_lora_to_model
from tunix_b200.models.config import ModelConfig
from tunix_b200.models.transformer import create_model
from tunix_b200.sft.dpo.dpo_trainer import DataInput, DPOTrainer, DPOTrainingConfig, TrainingInput, dpo_loss_fn
from tests.test_sampler_cpu import CharTok


def _cfg():
    return ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2,
                                            head_dim=16, num_kv_heads=1)


def _tok_batch(B=4, P=6, R=5, seed=0):
    g = np.random.default_rng(seed)
    pm = np.ones((B, P), np.int32)
    pm[0, :2] = 0
    cm = np.ones((B, R), np.int32)
    cm[1, 3:] = 0
    return TrainingInput(g.integers(1, 64, (B, P)), pm, g.integers(1, 64, (B, R)), cm, g.integers(1, 64, (B, R)),
                         np.ones((B, R), np.int32))


def test_dpo_initial_loss_is_log2_and_decreases():
    model, ref = create_model(_cfg(), seed=0), create_model(_cfg(), seed=0)
    tc = DPOTrainingConfig(eval_every_n_steps=100, max_steps=8, beta=0.1, pbar_description=None)
    tr = DPOTrainer(model, ref, optim.AdamW(5e-3, weight_decay=0.0), tc)
    batch = _tok_batch()
    tr.train([batch] * 8)
    hist = tr.metrics_logger.get_metric_history("", "loss", "train")
    assert abs(hist[0] - math.log(2)) < 1e-4           # policy == reference at step 0
    assert hist[-1] < hist[0]
    assert tr.metrics_logger.get_metric("", "rewards/accuracy", "train") > 0.4


def test_lora_policy_uses_frozen_backbone_as_reference():
    model = create_model(_cfg(), seed=0)
    apply_lora_to_model(model, LoraProvider(module_path=r".*(q_proj|v_proj|o_proj|k_proj|gate_proj|up_proj|down_proj)",
                                            rank=4, alpha=8.0))
    tc = DPOTrainingConfig(eval_every_n_steps=100, max_steps=2, pbar_description=None)
    tr = DPOTrainer(model, None, optim.AdamW(1e-2), tc)
    ex = tr._prepare_inputs(_tok_batch())
    assert ex.ref_chosen_logps is not None
    out = dpo_loss_fn(model, ex)
    assert abs(out.loss.value().item() - math.log(2)) < 1e-4


def test_orpo_and_string_inputs():
    model = create_model(_cfg(), seed=0)
    tc = DPOTrainingConfig(eval_every_n_steps=100, max_steps=2, algorithm="orpo", max_prompt_length=8,
                           max_response_length=6, pbar_description=None)
    tr = DPOTrainer(model, None, optim.AdamW(1e-3), tc, tokenizer=CharTok())
    tr.train([DataInput(["ab", "cde"], ["good", "fine"], ["bad", "no"])] * 2)
    assert tr.metrics_logger.metric_exists("", "odds_ratio", "train")
    assert tr.metrics_logger.metric_exists("", "sft_loss", "train")
