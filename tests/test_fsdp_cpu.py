"""Sharded optimizer logic on CPU ranks (gloo): 2 ranks with half the batch each == 1 rank with the full batch."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _train(rank, world, port, out):
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
                                           head_dim=32, num_kv_heads=1)
    model = create_model(cfg, seed=0)
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, 256, (4, 24), generator=g)
    mask = torch.ones(4, 24)
    mask[0, :10] = 0
    opt = (fsdp.ShardedAdamW(1e-2, weight_decay=0.01, max_grad_norm=0.5) if world > 1
           else optim.AdamW(1e-2, weight_decay=0.01, max_grad_norm=0.5))
    tc = TrainingConfig(eval_every_n_steps=1000, max_steps=3, pbar_description=None)
    tr = PeftTrainer(model, opt, tc)
    tr.train([TrainingInput(toks, mask)] * 3)
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
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
