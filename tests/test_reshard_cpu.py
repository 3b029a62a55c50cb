"""Weight reshard planning and the send / recv execution on CPU ranks (gloo)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tunix_b200.rl import reshard as rs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_plan_covers_rectangle_from_mixed_shards():
    full = (8, 12)
    srcs = [(0, rs.TensorSpec(full, (0, 4), (0, 12))), (1, rs.TensorSpec(full, (4, 8), (0, 12)))]
    dst = rs.TensorSpec(full, (2, 7), (4, 12))
    blocks = rs.plan_blocks("w", dst, 0, srcs)
    cover = torch.zeros(5, 8)
    for b in blocks:
        cover[b.dst_rc[0]:b.dst_rc[0] + b.rows, b.dst_rc[1]:b.dst_rc[1] + b.cols] += 1
    assert torch.all(cover == 1)
    assert {b.src_rank for b in blocks} == {0, 1}
    assert rs.kv_rows_for(num_kv_heads=2, head_dim=4, tp=4, tp_rank=3) == (4, 8)
    assert rs.kv_rows_for(num_kv_heads=8, head_dim=4, tp=2, tp_rank=1) == (16, 32)


def _run(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    full = {"a.weight": torch.randn(8, 6), "b.weight": torch.randn(4, 8), "norm.weight": torch.randn(6)}
    # ranks 0, 1: trainers (a: row shards, b: column shards, norm: whole); rank 2: rollout wants everything whole
    if rank < 2:
        a = full["a.weight"][rank * 4:(rank + 1) * 4].clone()
        a.shard_spec = (0, rank, 2)
        b = full["b.weight"][:, rank * 4:(rank + 1) * 4].clone()
        b.shard_spec = (1, rank, 2)
        src, dst = {"a.weight": a, "b.weight": b, "norm.weight": full["norm.weight"].clone()}, {}
    else:
        src, dst = {}, {n: torch.zeros_like(t) for n, t in full.items()}
        dst["head.weight"] = torch.zeros_like(full["a.weight"])            # tied: filled from a.weight
    r = rs.WeightReshard(src, dst, key_map=lambda n: "a.weight" if n == "head.weight" else n)
    r.run()
    if rank == 2:
        ok = all(torch.allclose(dst[n], full[n]) for n in full) and torch.allclose(dst["head.weight"], full["a.weight"])
        torch.save(torch.tensor(ok), out)
    dist.barrier()
    dist.destroy_process_group()


def test_sendrecv_reshard_three_ranks(tmp_path):
    out = str(tmp_path / "ok.pt")
    mp.spawn(_run, args=(3, 29747, out), nprocs=3, join=True)
    assert bool(torch.load(out))


def test_lora_merge_matches_formula():
    from tunix_b200.models.transformer import Linear
    lin = Linear(16, 8, False, torch.float32, None)
    torch.nn.init.normal_(lin.weight)
    lin.lora_a = torch.nn.Parameter(torch.randn(4, 16))
    lin.lora_b = torch.nn.Parameter(torch.randn(8, 4))
    lin.lora_scale = 0.5
    w = rs.merged_weight(lin)
    assert torch.allclose(w, lin.weight + 0.5 * lin.lora_b @ lin.lora_a, atol=1e-5)
