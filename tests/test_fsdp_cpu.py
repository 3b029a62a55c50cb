"""Sharded optimizer logic on CPU ranks (gloo): 2 ranks with half the batch each == 1 rank with the full batch."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _train(rank, world, port, out, variant="full"):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    from tunix_b200 import optim
    from tunix_b200.common.configs import TrainingConfig
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.parallel import fsdp
    from tunix_b200.sft.peft_trainer import PeftTrainer, TrainingInput
    torch.manual_seed(0)
    cfg = ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=256, embed_dim=64, hidden_dim=128, num_heads=2,
                                           head_dim=32, num_kv_heads=1, qkv_bias=variant != "full")
    model = create_model(cfg, seed=0)
    if variant == "lora":
        from tunix_b200.lora import LoraProvider, apply_lora_to_model
        apply_lora_to_model(model, LoraProvider(rank=4, alpha=8.0))
        with torch.no_grad():
            for n_, p_ in model.named_parameters():
                if n_.endswith("lora_b"):
                    p_.normal_(0.0, 0.05, generator=torch.Generator().manual_seed(11))
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, 256, (4, 24), generator=g)
    mask = torch.ones(4, 24)
    mask[0, :10] = 0
    opt = (fsdp.ShardedAdamW(1e-2, weight_decay=0.01, max_grad_norm=0.5) if world > 1
           else optim.AdamW(1e-2, weight_decay=0.01, max_grad_norm=0.5))
    tc = TrainingConfig(eval_every_n_steps=1000, max_steps=3, pbar_description=None)
    tr = PeftTrainer(model, opt, tc)
    tr.train([TrainingInput(toks, mask)] * 3)
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters() if p.requires_grad])
    if rank == 0:
        torch.save(flat, out)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def test_two_gloo_ranks_match_single_process(tmp_path):
    single, double = str(tmp_path / "s.pt"), str(tmp_path / "d.pt")
    _train(0, 1, 0, single)
    mp.spawn(_train, args=(2, 29731, double), nprocs=2, join=True)
    a, b = torch.load(single), torch.load(double)
    assert torch.allclose(a, b, atol=2e-5, rtol=1e-4), (a - b).abs().max()


@pytest.mark.parametrize("variant", ["bias", "lora"])
def test_two_gloo_ranks_match_single_process_with_biases_and_adapters(tmp_path, variant):
    """Bias and adapter gradients do not come from the wgrad epilogue; they must reach the sharded update too."""
    single, double = str(tmp_path / "s.pt"), str(tmp_path / "d.pt")
    _train(0, 1, 0, single, variant)
    mp.spawn(_train, args=(2, 29733 if variant == "bias" else 29735, double, variant), nprocs=2, join=True)
    a, b = torch.load(single), torch.load(double)
    assert torch.allclose(a, b, atol=2e-5, rtol=1e-4), (a - b).abs().max()


def test_flag_barrier_protocol_model_with_threads_as_ranks():
    """The device barrier's protocol restated on the host: nobody leaves barrier k before everybody entered it,
    under random schedules, with slots interleaved, across the 32-bit epoch wrap; a rank that stays away costs the
    others a bounded wait and a status that names it."""
    import random
    import threading
    import time
    from tunix_b200.parallel.protocol_model import ST_TIMEOUT_FLAG, FlagBarrierModel, _not_older, run_ranks
    assert _not_older(5, 5) and _not_older(6, 5) and not _not_older(4, 5)
    assert _not_older(2, 0xFFFFFFFE) and not _not_older(0xFFFFFFFE, 2)           # across the wrap
    for world, start in ((2, 0), (4, 0), (8, 0xFFFFFFF0)):
        model = FlagBarrierModel(world, slots=3)
        if start:
            model.set_epoch(start)
        rounds = 40
        entered = [[0] * world for _ in range(rounds)]
        lock = threading.Lock()

        def body(rank, model=model, entered=entered, world=world):
            rng = random.Random(rank)
            jitter = lambda: time.sleep(rng.random() * 2e-4) if rng.random() < 0.3 else None
            for k in range(rounds):
                with lock:
                    entered[k][rank] = 1
                assert model.wait(rank, slot=k % 3, timeout_s=20.0, yield_fn=jitter)
                with lock:
                    assert sum(entered[k]) == world, (k, rank)        # everybody had entered before anyone left
            return True
        assert all(run_ranks(world, body))
        assert not model.status.any()
    # rank 2 never joins the second barrier: the others give up after the limit and name it
    model = FlagBarrierModel(3)

    def body(rank):
        assert model.wait(rank, timeout_s=10.0)
        if rank == 2:
            return "left"
        return model.wait(rank, timeout_s=0.2)
    t0 = time.monotonic()
    assert run_ranks(3, body) == [False, False, "left"] and time.monotonic() - t0 < 5
    assert model.status[0].tolist() == [ST_TIMEOUT_FLAG, 2, 2] and model.status[1].tolist() == [ST_TIMEOUT_FLAG, 2, 2]
    assert model.status[2, 0] == 0
    # a late rank is not an absent one: the barrier completes once it shows up
    model = FlagBarrierModel(2)

    def late(rank):
        if rank == 1:
            time.sleep(0.15)
        return model.wait(rank, timeout_s=5.0)
    assert run_ranks(2, late) == [True, True]
