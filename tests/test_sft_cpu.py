"""CPU end-to-end: tiny Llama LoRA SFT through PeftTrainer (the CPU correctness config)."""
import math

import numpy as np
import torch

from tunix_b200 import optim
from tunix_b200.common.configs import TrainingConfig
from tunix_b200.lora import LoraProvider, apply_lora_to_model, is_lora_param_name
from tunix_b200.models.config import ModelConfig
from tunix_b200.models.transformer import create_model
from tunix_b200.sft.peft_trainer import PeftTrainer, TrainingInput, _default_loss_fn


def _batches(n, seed=1, B=4, T=128, vocab=1024):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        toks = torch.randint(0, vocab, (B, T), generator=g)
        mask = torch.zeros(B, T)
        mask[:, T - 64:] = 1
        out.append(TrainingInput(toks, mask))
    return out


def test_tiny_llama_lora_sft_loss_decreases(tmp_path):
    cfg = ModelConfig.tiny_llama()
    model = create_model(cfg, seed=0)
    apply_lora_to_model(model, LoraProvider(module_path=r".*(q_proj|v_proj)", rank=8, alpha=16.0))
    base_before = {n: p.detach().clone() for n, p in model.named_parameters() if not is_lora_param_name(n)}
    tc = TrainingConfig(eval_every_n_steps=1000, max_steps=20, checkpoint_root_directory=str(tmp_path / "ckpt"),
                        pbar_description=None)
    trainer = PeftTrainer(model, optim.AdamW(1e-3, weight_decay=0.0), tc)
    batch = _batches(1)[0]
    trainer.train([batch] * 20)
    hist = trainer.metrics_logger.get_metric_history("", "loss", "train")
    assert len(hist) == 20
    assert hist[0] > hist[-1]
    assert abs(hist[0] - math.log(1024)) < 0.2
    for n, p in model.named_parameters():
        if not is_lora_param_name(n):
            assert torch.equal(p, base_before[n]), n
    # resume: a new trainer on the same directory starts at step 20
    model2 = create_model(cfg, seed=0)
    apply_lora_to_model(model2, LoraProvider(module_path=r".*(q_proj|v_proj)", rank=8, alpha=16.0))
    tr2 = PeftTrainer(model2, optim.AdamW(1e-3, weight_decay=0.0), tc)
    assert tr2.train_steps == 20
    for (n, p), (_, q) in zip(model.named_parameters(), model2.named_parameters()):
        if is_lora_param_name(n):
            assert torch.allclose(p, q), n
    tr2.close()


def test_grad_accumulation_matches_full_batch():
    cfg = ModelConfig.tiny_llama().replace(num_layers=1)
    batches = _batches(1, B=4, T=32)
    full = batches[0]
    # unequal masks so that token-weighted averaging matters
    full.input_mask[0, :20] = 1
    halves = [TrainingInput(full.input_tokens[:2], full.input_mask[:2]),
              TrainingInput(full.input_tokens[2:], full.input_mask[2:])]
    results = []
    for data, accum in ((([full]), 1), (halves, 2)):
        model = create_model(cfg, seed=0)
        tc = TrainingConfig(eval_every_n_steps=1000, max_steps=1, gradient_accumulation_steps=accum,
                            pbar_description=None)
        tr = PeftTrainer(model, optim.SGD(0.1), tc)
        tr.train(data)
        results.append(torch.cat([p.detach().reshape(-1) for p in model.parameters()]))
    assert torch.allclose(results[0], results[1], atol=1e-5, rtol=1e-4)


def test_default_loss_matches_manual_cross_entropy():
    cfg = ModelConfig.tiny_llama().replace(num_layers=1)
    model = create_model(cfg, seed=0)
    b = _batches(1, B=2, T=16)[0]
    out = _default_loss_fn(model, b.input_tokens, b.input_mask)
    logits, _ = model(b.input_tokens)
    lsm = torch.log_softmax(logits[:, :-1].float(), -1)
    nll = -lsm.gather(-1, b.input_tokens[:, 1:, None])[..., 0]
    ref = (nll * b.input_mask[:, 1:]).sum() / b.input_mask[:, 1:].sum()
    assert torch.allclose(out.loss.value(), ref, atol=1e-5)


def test_step_time_and_throughput_metrics_are_logged():
    import numpy as np
    import torch
    from tunix_b200 import optim
    from tunix_b200.common.configs import TrainingConfig
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.sft.peft_trainer import PeftTrainer, TrainingInput
    cfg = ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2, head_dim=16, num_kv_heads=1)
    model = create_model(cfg, seed=0)
    tr = PeftTrainer(model, optim.AdamW(1e-3), TrainingConfig(eval_every_n_steps=10 ** 9, max_steps=4, gradient_accumulation_steps=2,
                                                               pbar_description=None))
    g = torch.Generator().manual_seed(0)
    data = [TrainingInput(torch.randint(1, 64, (2, 8), generator=g), torch.ones(2, 8, dtype=torch.int32)) for _ in range(8)]
    tr.train(data)
    lg = tr.metrics_logger
    times = lg.get_metric_history("", "step_time_sec", "train")
    assert len(times) == 3 and (times > 0).all()                       # every step after the first has a predecessor to time against
    np.testing.assert_allclose(lg.get_metric_history("", "steps_per_sec", "train"), 1.0 / times)
    n = sum(p.numel() for p in model.parameters())
    np.testing.assert_allclose(lg.get_metric_history("", "tflops_per_step", "train"), 6.0 * n * 32 / times / 1e12, rtol=1e-6)
