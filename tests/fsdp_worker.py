"""Worker for the multi-GPU sharded-optimizer test (run under torch.distributed.run)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    comm = sys.argv[1] if len(sys.argv) > 1 else "p2p"
    out_path = sys.argv[2] if len(sys.argv) > 2 else None
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from tunix_b200 import _lib, optim
    from tunix_b200.common.configs import TrainingConfig
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.parallel import fsdp
    from tunix_b200.sft.peft_trainer import PeftTrainer, TrainingInput

    cfg = ModelConfig(family="llama3", num_layers=3, vocab_size=4096, embed_dim=512, hidden_dim=1024, num_heads=4,
                      head_dim=128, num_kv_heads=2, dtype=torch.bfloat16, max_position=512)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, 4096, (2 * world, 256), generator=g)
    mask = torch.ones(2 * world, 256)
    mask[:, :64] = 0

    def run(opt, shard):
        model = create_model(cfg, device=dev, seed=0)
        tc = TrainingConfig(eval_every_n_steps=10 ** 9, max_steps=3, pbar_description=None)
        tr = PeftTrainer(model, opt, tc)
        if not shard:
            tr._shard_and_move = lambda b: TrainingInput(b.input_tokens.to(dev), b.input_mask.to(dev))
        tr.train([TrainingInput(toks, mask)] * 3)
        torch.cuda.synchronize()
        _lib.raise_if_kernel_error()
        losses = tr.metrics_logger.get_metric_history("", "loss", "train").tolist()
        return torch.cat([p.detach().float().reshape(-1) for p in model.parameters()]), losses

    sharded, l_sh = run(fsdp.ShardedAdamW(1e-3, weight_decay=0.0, max_grad_norm=1.0, comm=comm), True)
    # oracle: every rank trains the full global batch alone
    single, l_si = run(optim.AdamW(1e-3, weight_decay=0.0, max_grad_norm=1.0), False)
    rel = ((sharded - single).norm() / single.norm()).item()
    # all ranks must hold identical parameters after the all-gather
    ref = sharded.clone()
    dist.broadcast(ref, 0)
    same = bool(torch.equal(ref, sharded))
    flags = torch.tensor([1.0 if same else 0.0], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0 and out_path:
        json.dump({"rel": rel, "same": bool(flags.item() == 1.0), "loss_sharded": l_sh, "loss_single": l_si},
                  open(out_path, "w"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
