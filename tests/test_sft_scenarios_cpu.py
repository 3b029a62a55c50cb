"""Trainer behaviour above the kernels, scenario by scenario (the situations the reference's trainer tests cover,
tests/sft/peft_trainer_test.py: accumulation equivalences, packed vs. unpacked, dtype preservation, hooks, custom
losses with aux metrics, checkpoint cadence, resume that skips consumed batches, adapter-only checkpoints)."""
import math
import os

import numpy as np
import pytest
import torch

from tunix_b200 import optim
from tunix_b200.common.configs import TrainingConfig
from tunix_b200.lora import LoraProvider, apply_lora_to_model, is_lora_param_name
from tunix_b200.models.config import ModelConfig
from tunix_b200.models.transformer import create_model
from tunix_b200.sft import hooks as hooks_lib
from tunix_b200.sft.peft_trainer import GradientAccumulator, PeftTrainer, TrainingInput, _default_loss_fn
from tunix_b200.sft.utils import LossOutput, WeightedMetric


def _cfg(**kw):
    return ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=128, embed_dim=32, hidden_dim=64, num_heads=2,
                                            head_dim=16, num_kv_heads=1, **kw)


def _data(B=8, T=24, seed=3, vocab=128):
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(0, vocab, (B, T), generator=g)
    mask = (torch.rand(B, T, generator=g) > 0.3).float()
    mask[:, 0] = 1
    return toks, mask


def _flat(model):
    return torch.cat([p.detach().reshape(-1).float() for p in model.parameters()])


def _tc(**kw):
    base = dict(eval_every_n_steps=10 ** 6, pbar_description=None)
    base.update(kw)
    return TrainingConfig(**base)


@pytest.mark.parametrize("K", [2, 4, 8])
def test_K_micro_batches_equal_one_batch_with_token_weighted_denominators(K):
    """Micro-batches with very different numbers of loss tokens: the update is sum(grad) / sum(tokens), not a mean of
    per-micro-batch means."""
    toks, mask = _data(B=8)
    mask[0, :] = 1                      # one long row, several short ones
    mask[5, 3:] = 0
    out = []
    for pieces in (1, K):
        model = create_model(_cfg(), seed=0)
        n = 8 // pieces
        data = [TrainingInput(toks[i * n:(i + 1) * n], mask[i * n:(i + 1) * n]) for i in range(pieces)]
        tr = PeftTrainer(model, optim.SGD(0.5), _tc(max_steps=1, gradient_accumulation_steps=pieces))
        tr.train(data)
        assert tr.train_steps == 1 and tr.iter_steps == pieces
        out.append(_flat(model))
    assert torch.allclose(out[0], out[1], atol=2e-6, rtol=1e-5)


def test_packed_rows_train_like_the_unpacked_sequences():
    """Two sequences packed into one row with segment ids and restarted positions give the update of the two rows."""
    cfg = _cfg()
    g = torch.Generator().manual_seed(5)
    a, b = torch.randint(0, 128, (1, 10), generator=g), torch.randint(0, 128, (1, 14), generator=g)

    def run(batch_kwargs):
        model = create_model(cfg, seed=0)
        tr = PeftTrainer(model, optim.SGD(0.3), _tc(max_steps=1))
        tr.gen_model_input_fn = lambda x: x
        tr.train([batch_kwargs])
        return _flat(model)
    # unpacked: two rows padded to 14, mask 0 on the padding
    toks = torch.zeros(2, 14, dtype=torch.long)
    toks[0, :10], toks[1] = a[0], b[0]
    mask = torch.zeros(2, 14)
    mask[0, :10], mask[1] = 1, 1
    seg = torch.where(mask > 0, torch.ones(2, 14, dtype=torch.int32), torch.zeros(2, 14, dtype=torch.int32))
    unpacked = run({"input_tokens": toks, "input_mask": mask, "segment_ids": seg})
    # packed: one row [a | b]; the first token of b is not a target of a's last token
    ptoks = torch.cat([a, b], 1)
    pseg = torch.cat([torch.full((1, 10), 1, dtype=torch.int32), torch.full((1, 14), 2, dtype=torch.int32)], 1)
    ppos = torch.cat([torch.arange(10), torch.arange(14)])[None].int()
    pmask = torch.ones(1, 24)
    pmask[0, 10] = 0                      # position 10 (b's first token) is predicted from a's last one: no loss there
    packed = run({"input_tokens": ptoks, "input_mask": pmask, "segment_ids": pseg, "positions": ppos})
    assert torch.allclose(unpacked, packed, atol=3e-6, rtol=1e-5)


@pytest.mark.parametrize("accum", [1, 3])
def test_parameters_and_optimizer_state_keep_their_dtypes(accum):
    model = create_model(_cfg(dtype=torch.bfloat16), seed=0)
    toks, mask = _data(B=3)
    tr = PeftTrainer(model, optim.AdamW(1e-2), _tc(max_steps=2, gradient_accumulation_steps=accum))
    tr.train([TrainingInput(toks[i:i + 1], mask[i:i + 1]) for i in range(3)] * 2)
    assert all(p.dtype == torch.bfloat16 for p in model.parameters())
    st = tr.optimizer._state_tensors()
    assert st["mu"].dtype == st["nu"].dtype == st["master"].dtype == torch.float32     # fp32 moments and master copy
    assert tr.optimizer.buffers.grad_flat.dtype == torch.float32                       # CPU / accumulation: fp32 sums
    assert tr.train_steps == 2


def test_gradient_accumulator_arithmetic():
    p = [torch.zeros(3, dtype=torch.bfloat16), torch.zeros(2, 2)]
    acc = GradientAccumulator(p)
    acc.add([torch.tensor([1.0, 2.0, 3.0]), torch.ones(2, 2)], denom=2.0)
    acc.add([torch.tensor([3.0, 2.0, 1.0]), None], denom=6.0)
    g = acc.get()
    assert g[0].dtype == torch.bfloat16 and torch.allclose(g[0].float(), torch.tensor([0.5, 0.5, 0.5]))
    assert torch.allclose(g[1], torch.full((2, 2), 0.125))
    acc.reset()
    assert all(float(x.abs().sum()) == 0 for x in acc.get())                           # zero denominator -> zero grads
    acc.add([torch.ones(3), torch.ones(2, 2)], denom=1.0)
    assert torch.allclose(acc.get()[1], torch.ones(2, 2))                              # no state leaks through reset


def test_hooks_fire_in_order_and_data_hooks_can_feed_the_loop():
    toks, mask = _data(B=4)
    events = []

    class H(hooks_lib.TrainingHooks):
        def on_train_start(self, ctx): events.append("start")
        def on_train_end(self, ctx): events.append("end")
        def on_train_step_start(self, ctx): events.append("s")
        def on_train_step_end(self, ctx, step, loss): events.append(("e", step, loss > 0))
        def on_eval_step_start(self, ctx): events.append("es")
        def on_eval_step_end(self, ctx, loss): events.append(("ee", loss > 0))

    class D(hooks_lib.DataHooks):
        def __init__(self): self.n = 0
        def load_next_train_batch(self, ctx):
            self.n += 1
            return TrainingInput(toks, mask) if self.n <= 3 else None
        def load_next_eval_batch(self, ctx):
            return None

    model = create_model(_cfg(), seed=0)
    tr = PeftTrainer(model, optim.AdamW(1e-3), _tc(max_steps=10)).with_training_hooks(H()).with_data_hooks(D())
    tr.train(None)
    assert tr.train_steps == 3 and events[0] == "start" and "end" in events
    assert events.count("s") == 3
    ends = [e for e in events if isinstance(e, tuple) and e[0] == "e"]
    assert [e[1] for e in ends] == [1, 2, 3][:len(ends)] and all(e[2] for e in ends)      # delayed by one step, flushed at close


def test_custom_loss_with_aux_metrics_and_plain_scalar_loss():
    toks, mask = _data(B=4)
    model = create_model(_cfg(), seed=0)

    def loss_fn(model, input_tokens, input_mask):
        out = _default_loss_fn(model, input_tokens, input_mask)
        return LossOutput(out.loss, aux={"tokens": WeightedMetric(input_mask.sum(), torch.tensor(1.0)), "const": 2.5})
    tr = PeftTrainer(model, optim.AdamW(1e-3), _tc(max_steps=2)).with_loss_fn(loss_fn, has_aux=True)
    tr.train([TrainingInput(toks, mask)] * 2)
    lg = tr.metrics_logger
    assert lg.get_metric_history("", "const", "train").tolist() == [2.5, 2.5]
    assert lg.get_metric_history("", "tokens", "train")[0] == float(mask.sum())
    # a loss function may also return a bare scalar: micro-batches are then averaged
    model2 = create_model(_cfg(), seed=0)
    tr2 = PeftTrainer(model2, optim.SGD(0.1), _tc(max_steps=1, gradient_accumulation_steps=2))
    tr2.with_loss_fn(lambda model, input_tokens, input_mask: _default_loss_fn(model, input_tokens, input_mask).loss.value())
    tr2.train([TrainingInput(toks[:2], mask[:2]), TrainingInput(toks[2:], mask[2:])])
    assert tr2.train_steps == 1 and len(tr2.metrics_logger.get_metric_history("", "loss", "train")) == 1


def test_checkpoint_cadence_retention_and_resume_skips_consumed_batches(tmp_path):
    toks, mask = _data(B=12)
    data = [TrainingInput(toks[i:i + 2], mask[i:i + 2]) for i in range(0, 12, 2)]      # 6 different batches
    ck = dict(checkpoint_root_directory=str(tmp_path / "ck"),
              checkpointing_options={"save_interval_steps": 2, "max_to_keep": 2, "enable_async_checkpointing": False})
    # uninterrupted: 6 steps
    m_full = create_model(_cfg(), seed=0)
    PeftTrainer(m_full, optim.AdamW(1e-2, weight_decay=0.0), _tc(max_steps=6)).train(data)
    # interrupted after 4 steps, then a new trainer over the SAME data resumes at 4 and trains on batches 5 and 6 only
    m1 = create_model(_cfg(), seed=0)
    t1 = PeftTrainer(m1, optim.AdamW(1e-2, weight_decay=0.0), _tc(max_steps=4, **ck))
    t1.train(data)
    assert sorted(int(d) for d in os.listdir(tmp_path / "ck")) == [2, 4]
    m2 = create_model(_cfg(), seed=1)                                                    # other weights: restore must win
    t2 = PeftTrainer(m2, optim.AdamW(1e-2, weight_decay=0.0), _tc(max_steps=6, **ck))
    assert t2.train_steps == 4
    seen = []
    orig = t2._train_step
    t2._train_step = lambda b, u: (seen.append(b.input_tokens.clone()), orig(b, u))[1]
    t2.train(data)
    assert t2.train_steps == 6 and len(seen) == 2 and torch.equal(seen[0].cpu(), data[4].input_tokens)
    assert torch.allclose(_flat(m2), _flat(m_full), atol=1e-6)
    assert sorted(int(d) for d in os.listdir(tmp_path / "ck")) == [4, 6]                 # the two latest are kept
    # asking not to resume starts from scratch
    t3 = PeftTrainer(create_model(_cfg(), seed=0), optim.AdamW(1e-2), _tc(max_steps=1, resume_from_checkpoint_on_init=False, **ck))
    assert t3.train_steps == 0


def test_lora_checkpoints_hold_adapters_only_and_restore_into_a_fresh_backbone(tmp_path):
    from tunix_b200.sft.checkpoint_manager import _flatten, _load_item
    toks, mask = _data(B=2)
    ck = dict(checkpoint_root_directory=str(tmp_path / "ck"),
              checkpointing_options={"save_interval_steps": 1, "enable_async_checkpointing": False})
    model = create_model(_cfg(), seed=0)
    apply_lora_to_model(model, LoraProvider(module_path=r".*(q_proj|down_proj)", rank=4, alpha=8.0))
    tr = PeftTrainer(model, optim.AdamW(1e-2, weight_decay=0.0), _tc(max_steps=2, **ck))
    tr.train([TrainingInput(toks, mask)] * 2)
    saved = {".".join(k): v for k, v in _flatten(_load_item(str(tmp_path / "ck" / "2" / "model_params"))).items()}
    assert saved and all(is_lora_param_name(n) for n in saved)
    fresh = create_model(_cfg(), seed=0)
    apply_lora_to_model(fresh, LoraProvider(module_path=r".*(q_proj|down_proj)", rank=4, alpha=8.0), seed=7)
    t2 = PeftTrainer(fresh, optim.AdamW(1e-2, weight_decay=0.0), _tc(max_steps=2, **ck))
    assert t2.train_steps == 2
    for (n, p), (_, q) in zip(model.named_parameters(), fresh.named_parameters()):
        assert torch.allclose(p, q), n


def test_reusing_a_trainer_continues_where_it_stopped_and_learning_rate_follows_the_schedule():
    toks, mask = _data(B=2)
    model = create_model(_cfg(), seed=0)
    sched = optim.warmup_cosine_decay_schedule(0.0, 1e-2, 2, 6, 0.0)
    tr = PeftTrainer(model, optim.AdamW(sched, weight_decay=0.0), _tc(max_steps=3))
    tr.is_managed_externally = True          # keep loggers open between calls
    tr.train([TrainingInput(toks, mask)] * 3)
    tr.config.max_steps = 5
    tr.is_managed_externally = False
    tr.train([TrainingInput(toks, mask)] * 5)
    lrs = tr.metrics_logger.get_metric_history("", "learning_rate", "train")
    assert tr.train_steps >= 5 and lrs[0] == 0.0 and math.isclose(lrs[2], 1e-2, rel_tol=1e-6) and lrs[-1] < lrs[2]


def _failing_rank_worker(rank, world, port, out):
    import os
    import sys
    import time
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from tunix_b200 import optim
    from tunix_b200.common.configs import TrainingConfig
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.parallel.watchdog import RankFailure
    from tunix_b200.sft.peft_trainer import PeftTrainer, TrainingInput
    cfg = ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2, head_dim=16, num_kv_heads=1)
    tr = PeftTrainer(create_model(cfg, seed=0), optim.AdamW(1e-3), TrainingConfig(eval_every_n_steps=10 ** 9, pbar_description=None,
                                                                                  rank_failure_timeout_s=0.8))
    g = torch.Generator().manual_seed(rank)

    def batches():
        for i in range(10 ** 6):
            if rank == 1 and i == 3:
                os._exit(0)                                  # the rank disappears between steps, nothing in flight
            time.sleep(0.05)
            yield {"input_tokens": torch.randint(1, 64, (2, 8), generator=g), "input_mask": torch.ones(2, 8, dtype=torch.int32),
                   "_is_local_shard": True}
    try:
        tr.train(batches())
        res = "finished"
    except RankFailure as e:
        res = ("rank failure", e.ranks, tr.train_steps)
    torch.save(res, out)
    os._exit(0)                                              # no collective teardown with a peer that is gone


def test_training_stops_cleanly_when_a_rank_disappears(tmp_path):
    import torch
    import torch.multiprocessing as mp
    out = str(tmp_path / "r0.pt")
    mp.spawn(_failing_rank_worker, args=(2, 29761, out), nprocs=2, join=True)
    kind, ranks, steps = torch.load(out)
    assert kind == "rank failure" and ranks == [1] and steps >= 3
