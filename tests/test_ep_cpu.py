"""Expert parallelism on CPU ranks (gloo): 2 ranks with half the experts and half the batch each == 1 rank."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    from tunix_b200 import optim
    from tunix_b200.common.configs import TrainingConfig
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.parallel import ep as ep_lib
    from tunix_b200.sft.peft_trainer import PeftTrainer, TrainingInput
    cfg = ModelConfig.tiny_llama().replace(num_layers=2, vocab_size=256, embed_dim=64, hidden_dim=128, num_heads=4, head_dim=16,
                                           num_kv_heads=2, num_experts=4, num_experts_per_tok=2, moe_hidden_dim=32)
    model = create_model(cfg, seed=0)
    if world > 1:
        ep_lib.shard_experts(model, ep_lib.EPContext(device="cpu"))
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, 256, (4, 24), generator=g)
    mask = torch.ones(4, 24)
    mask[2, :5] = 0
    tr = PeftTrainer(model, optim.AdamW(1e-2, weight_decay=0.01, max_grad_norm=0.5),
                     TrainingConfig(eval_every_n_steps=1000, max_steps=3, pbar_description=None))
    tr.train([TrainingInput(toks, mask)] * 3)
    torch.save({n: p.detach().clone() for n, p in model.named_parameters()}, f"{out}.{rank}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def test_expert_parallel_training_matches_single_process(tmp_path):
    _run(0, 1, 0, str(tmp_path / "one"))
    mp.spawn(_run, args=(2, 29745, str(tmp_path / "two")), nprocs=2, join=True)
    one = torch.load(str(tmp_path / "one") + ".0")
    parts = [torch.load(str(tmp_path / "two") + f".{r}") for r in range(2)]
    for n, w in one.items():
        got = torch.cat([p[n] for p in parts], 0) if parts[0][n].shape != w.shape else parts[0][n]
        assert torch.allclose(got, w, atol=5e-5, rtol=2e-4), (n, (got - w).abs().max())


def test_plan_sizes_buffers_by_received_rows():
    """The routing plan bounds what a rank receives by its actual (128-padded) row count, not by the worst case."""
    import torch
    from tunix_b200.parallel.ep import _Plan

    class Ctx:
        def __init__(self, world, rank):
            self.world, self.rank = world, rank
    W, T, k, E = 4, 50, 2, 8
    g = torch.Generator().manual_seed(0)
    idx_all = torch.randint(0, E, (W * T, k), generator=g, dtype=torch.int32)
    total = 0
    for r in range(W):
        p = _Plan(idx_all, E, Ctx(W, r))
        counts = torch.bincount(idx_all.reshape(-1).long(), minlength=E).view(W, E // W)[r]
        want = int(((counts + 127) // 128 * 128).sum())
        assert p.rows == max(128, want) and p.rows <= p.max_rows and p.src_rank.numel() == p.rows
        assert int((p.src_rank >= 0).sum()) == int(counts.sum()) and int(p.seg_off[-1]) == want
        mine = p.own_dest < p.rows
        assert int(mine.sum()) == int(counts.sum()) and int(p.own_dest.max()) <= p.rows
        # every owned slot is the row the plan says it is: (source rank, token) recovered from the slot index
        slot = torch.arange(W * T * k)[mine]
        assert torch.equal(p.src_rank[p.own_dest[mine]].long(), slot // (T * k))
        assert torch.equal(p.src_row[p.own_dest[mine]].long(), (slot // k) % T)
        total += int(counts.sum())
    assert total == W * T * k


def test_plan_with_fixed_capacity_drops_overflow_and_flags_it():
    """Fixed-capacity plans need no read-back: with room to spare they equal the exact plan; when an owner would
    receive more rows than the capacity, the slots past it are dropped on both sides and the overflow flag is set."""
    import pytest
    import torch
    from tunix_b200.parallel.ep import EPContext, _Plan

    def ctx(world, rank, cf=None):
        c = EPContext.__new__(EPContext)
        c.world, c.rank, c.capacity_factor, c.overflow = world, rank, cf, None
        return c
    W, T, k, E = 2, 96, 2, 4
    g = torch.Generator().manual_seed(1)
    idx_all = torch.randint(0, E, (W * T, k), generator=g, dtype=torch.int32)
    for r in range(W):
        exact = _Plan(idx_all, E, ctx(W, r))
        roomy_ctx = ctx(W, r, cf=4.0)
        roomy = _Plan(idx_all, E, roomy_ctx)
        assert roomy.rows >= exact.rows and not bool(roomy_ctx.overflow)
        assert torch.equal(roomy.dst_rank, exact.dst_rank) and torch.equal(roomy.dst_pos, exact.dst_pos)
        assert torch.equal(roomy.seg_off, exact.seg_off) and torch.equal(roomy.counts, exact.counts)
        assert torch.equal(roomy.src_rank[:exact.rows], exact.src_rank) and int((roomy.src_rank[exact.rows:] >= 0).sum()) == 0
    # everything routed to expert 0 (rank 0): 2048 rows wanted, capacity 0.5 * 1024 + 2 * 128 = 768
    T2 = 512
    skew = torch.zeros(W * T2, k, dtype=torch.int32)
    c0 = ctx(W, 0, cf=0.5)
    p0 = _Plan(skew, E, c0)
    assert p0.rows == 768 and bool(c0.overflow)
    assert p0.seg_off.tolist() == [0, 768, 768] and p0.counts.tolist() == [768, 0]
    assert int((p0.src_rank >= 0).sum()) == 768                       # the owner fills exactly its capacity
    kept = (p0.dst_rank >= 0)
    c1 = ctx(W, 1, cf=0.5)
    p1 = _Plan(skew, E, c1)
    assert int(kept.sum()) + int((p1.dst_rank >= 0).sum()) == 768      # the sources agree on which slots survive
    assert int(p0.dst_pos[kept].max()) < 768
    with pytest.raises(RuntimeError):
        c0.raise_if_overflow()
    c0.raise_if_overflow()                                             # cleared after it was reported
