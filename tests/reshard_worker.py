"""Worker of tests/test_reshard_gpu.py: rank 0 trains (LoRA on one layer), rank 1 serves; weights move over P2P."""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    out_path = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    dev = torch.device("cuda", torch.cuda.current_device())
    from tunix_b200 import _lib
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.rl import reshard as rs
    big = len(sys.argv) > 2 and sys.argv[2] == "bench"
    cfg = ModelConfig(family="llama3", num_layers=4 if big else 2, vocab_size=32000 if big else 512,
                      embed_dim=4096 if big else 256, hidden_dim=14336 if big else 512, num_heads=32 if big else 4,
                      head_dim=128 if big else 64, num_kv_heads=8 if big else 2, dtype=torch.bfloat16, max_position=256)
    model = create_model(cfg, device=dev, seed=rank)          # different weights on the two ranks
    res = {}
    if rank == 0:
        lin = model.layers[0].self_attn.q_proj
        lin.lora_a = torch.nn.Parameter(torch.randn(16, lin.weight.shape[1], device=dev).to(torch.bfloat16) * 0.1)
        lin.lora_b = torch.nn.Parameter(torch.randn(lin.weight.shape[0], 16, device=dev).to(torch.bfloat16) * 0.1)
        lin.lora_scale, lin.lora_enabled = 2.0, True
        src, dst = rs.model_sources(model), {}
        want = {n: t.detach().float().cpu() for n, t in src.items()}
    else:
        src, dst = {}, {n: p.data for n, p in model.named_parameters()}
    r = rs.WeightReshard(src, dst, device=dev)
    res["fused"] = r.fused
    r.run()
    _lib.raise_if_kernel_error()
    torch.cuda.synchronize()
    if big:
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(3):
            r.run()
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / 3
        res["seconds"] = dt
        res["gbytes"] = r.bytes_pulled / 1e9
        res["gb_per_s_incl_staging"] = r.bytes_pulled / 1e9 / dt if rank == 1 else 0.0
    # rank 1 sends what it received back for the comparison on rank 0
    names = sorted(n for n, _ in model.named_parameters() if "lora_" not in n)
    worst = 0.0
    for n in names[:40]:
        t = dict(model.named_parameters())[n].data if rank == 1 else torch.empty_like(dict(model.named_parameters())[n].data)
        dist.broadcast(t, src=1)
        if rank == 0:
            worst = max(worst, float((t.float().cpu() - want[n]).abs().max()))
    res["max_abs_diff"] = worst
    allres = [None] * world
    dist.all_gather_object(allres, res)
    if rank == 0:
        json.dump(allres, open(out_path, "w"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
