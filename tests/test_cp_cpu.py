"""Context parallelism (the sequence axis sharded over a group) on CPU ranks (gloo): a model whose ranks each keep half
(a quarter) of every sequence trains like the whole one, packed segments and left padding included."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(rank, world, port, out, mesh_shape):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    from tunix_b200 import optim
    from tunix_b200.common.configs import TrainingConfig
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.parallel import mesh as mesh_lib, strategy
    from tunix_b200.sft.peft_trainer import PeftTrainer
    cfg = ModelConfig.tiny_llama().replace(num_layers=2, vocab_size=256, embed_dim=64, hidden_dim=128, num_heads=4,
                                           head_dim=16, num_kv_heads=2)
    model = create_model(cfg, seed=0)
    opt = optim.AdamW(1e-2, weight_decay=0.01, max_grad_norm=0.5)
    mesh = None
    if world > 1:
        mesh = mesh_lib.create_mesh(mesh_shape, ("fsdp", "sp"))
        mesh_lib.set_mesh(mesh)
        opt, plan = strategy.apply_parallelism(model, opt, mesh, device="cpu")
        assert plan.kind == "sp" and model.cp.world == mesh_shape[1]
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, 256, (4, 24), generator=g)
    mask = torch.ones(4, 24)
    mask[1, :7] = 0                                            # left padding
    seg = torch.ones(4, 24, dtype=torch.int32)
    seg[2, 10:] = 2                                            # a packed row: two documents, one boundary inside a slice
    seg[1, :7] = 0
    pos = torch.arange(24)[None].expand(4, 24).clone()
    pos[2, 10:] -= 10
    tr = PeftTrainer(model, opt, TrainingConfig(eval_every_n_steps=1000, max_steps=3, pbar_description=None))
    batch = {"input_tokens": toks, "input_mask": mask, "positions": pos, "segment_ids": seg}
    tr.train([batch] * 3)
    torch.save({"params": {n: p.detach().clone() for n, p in model.named_parameters()},
                "loss": [float(x) for x in tr.metrics_logger.get_metric_history("", "loss", "train")]}, f"{out}.{rank}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("world,mesh_shape,port", [(2, (1, 2), 29761), (4, (2, 2), 29763)])
def test_context_parallel_training_matches_single_process(tmp_path, world, mesh_shape, port):
    base = str(tmp_path / "one")
    _run(0, 1, 0, base, None)
    mp.spawn(_run, args=(world, port, str(tmp_path / "many"), mesh_shape), nprocs=world, join=True)
    one = torch.load(base + ".0")
    parts = [torch.load(str(tmp_path / "many") + f".{r}") for r in range(world)]
    for n, w in one["params"].items():
        for p in parts[1:]:
            assert torch.allclose(parts[0]["params"][n], p["params"][n], atol=1e-6), n      # replicas stay in step
        got = parts[0]["params"][n]
        assert torch.allclose(got, w, atol=3e-5, rtol=1e-4), (n, (got - w).abs().max())
    # a rank logs the loss of its own slice of the sequences; the slices' losses bracket the full-sequence loss
    assert len(one["loss"]) == 3 and all(len(p["loss"]) == 3 for p in parts)
    for step in range(3):
        local = [p["loss"][step] for p in parts]
        assert min(local) - 1e-4 <= one["loss"][step] <= max(local) + 1e-4, (one["loss"][step], local)
