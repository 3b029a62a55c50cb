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
    variant = sys.argv[3] if len(sys.argv) > 3 else "full"     # full | bias | lora
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
                      head_dim=128, num_kv_heads=2, dtype=torch.bfloat16, max_position=512,
                      qkv_bias=variant in ("bias", "lora"))
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, 4096, (2 * world, 256), generator=g)
    mask = torch.ones(2 * world, 256)
    mask[:, :64] = 0

    sizes = []

    def build():
        model = create_model(cfg, device=dev, seed=0)
        if variant == "lora":
            from tunix_b200.lora import LoraProvider, apply_lora_to_model
            apply_lora_to_model(model, LoraProvider(rank=8, alpha=16.0))
            with torch.no_grad():      # a zero lora_b would give lora_a no gradient in the first step
                gl = torch.Generator(device=dev).manual_seed(7)
                for n_, p_ in model.named_parameters():
                    if n_.endswith("lora_b"):
                        p_.normal_(0.0, 0.02, generator=gl)
                    p_.requires_grad_("lora_" in n_)
        return model

    def run(opt, shard):
        model = build()
        tc = TrainingConfig(eval_every_n_steps=10 ** 9, max_steps=3, pbar_description=None)
        tr = PeftTrainer(model, opt, tc)
        if not shard:
            tr._shard_and_move = lambda b: TrainingInput(b.input_tokens.to(dev), b.input_mask.to(dev))
        tr.train([TrainingInput(toks, mask)] * 3)
        torch.cuda.synchronize()
        _lib.raise_if_kernel_error()
        losses = tr.metrics_logger.get_metric_history("", "loss", "train").tolist()
        sizes[:] = [(n, p.numel()) for n, p in model.named_parameters() if p.requires_grad]
        trained = [p for p in model.parameters() if p.requires_grad]
        return torch.cat([p.detach().float().reshape(-1) for p in trained]), losses

    sharded, l_sh = run(fsdp.ShardedAdamW(1e-3, weight_decay=0.0, max_grad_norm=1.0, comm=comm), True)
    # oracle: every rank trains the full global batch alone
    single, l_si = run(optim.AdamW(1e-3, weight_decay=0.0, max_grad_norm=1.0), False)
    rel = ((sharded - single).norm() / single.norm()).item()
    # how far training moved the parameters: a gradient that never arrives shows up as a large share of this
    base = torch.cat([p.detach().float().reshape(-1) for p in build().parameters() if p.requires_grad])
    moved, off = 0.0, 0
    for n_, k in sizes:          # per tensor, so that a small tensor (a bias, an adapter) cannot hide in the total
        sl = slice(off, off + k)
        upd = (single[sl] - base[sl]).norm()
        if upd > 0:
            moved = max(moved, ((sharded[sl] - single[sl]).norm() / upd).item())
        off += k
    # all ranks must hold identical parameters after the all-gather
    ref = sharded.clone()
    dist.broadcast(ref, 0)
    same = bool(torch.equal(ref, sharded))
    flags = torch.tensor([1.0 if same else 0.0], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0 and out_path:
        json.dump({"rel": rel, "rel_to_update": moved, "same": bool(flags.item() == 1.0), "loss_sharded": l_sh, "loss_single": l_si},
                  open(out_path, "w"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
