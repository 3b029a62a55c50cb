"""Worker of tests/test_ep_gpu.py: launched with torch.distributed.run, one rank per GPU."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-6)).item()


def main():
    out_path = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    dev = torch.device("cuda", torch.cuda.current_device())
    from tunix_b200 import _lib
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import MoELayer
    from tunix_b200.ops import moe as moe_ops
    from tunix_b200.parallel import ep as ep_lib
    ep = ep_lib.EPContext(device=dev)
    res = {"fused": ep.fused}
    cfg = ModelConfig(family="qwen3", num_layers=1, vocab_size=64, embed_dim=256, hidden_dim=256, num_heads=2, head_dim=64,
                      num_kv_heads=1, dtype=torch.bfloat16, num_experts=8, num_experts_per_tok=2, moe_hidden_dim=128)
    torch.manual_seed(0)
    full = MoELayer(cfg, device=dev)
    for p in full.parameters():
        p.data.normal_(0, 0.05)
    part = MoELayer(cfg, device=dev)
    part.load_state_dict(full.state_dict())

    class Holder(torch.nn.Module):
        def __init__(self, m):
            super().__init__()
            self.m = m
    ep_lib.shard_experts(Holder(part), ep)
    T, D, E, k = 200, 256, 8, 2
    torch.manual_seed(11)
    x_all = (torch.randn(world * T, D, device=dev) * 0.5).to(torch.bfloat16)
    logits = torch.randn(world * T, E, device=dev)
    w_all, idx_all = torch.topk(torch.softmax(logits, -1), k, -1)
    dout_all = torch.randn(world * T, D, device=dev).to(torch.bfloat16)
    sl = slice(rank * T, (rank + 1) * T)
    # whole layer, all tokens, one GPU
    xr = x_all.clone().requires_grad_()
    wr = w_all.clone().requires_grad_()
    ref = moe_ops.experts(xr, wr, idx_all, full.gate_proj, full.up_proj, full.down_proj)
    ref.backward(dout_all)
    # expert parallel, this rank's tokens
    for rep in range(2):
        for p in part.parameters():
            p.grad = None
        xs = x_all[sl].clone().requires_grad_()
        ws_ = w_all[sl].clone().requires_grad_()
        out = ep_lib.expert_parallel_forward(part, xs, ws_, idx_all[sl])
        out.backward(dout_all[sl])
        _lib.raise_if_kernel_error()
        n = E // world
        res[f"out_{rep}"] = rel(out, ref[sl])
        res[f"dx_{rep}"] = rel(xs.grad, xr.grad[sl])
        res[f"dw_{rep}"] = rel(ws_.grad, wr.grad[sl])
        res[f"dgate_{rep}"] = rel(part.gate_proj.grad, full.gate_proj.grad[rank * n:(rank + 1) * n])
        res[f"ddown_{rep}"] = rel(part.down_proj.grad, full.down_proj.grad[rank * n:(rank + 1) * n])
    # the same with fixed-capacity receive buffers (no read-back in the routing plan): identical results while the
    # capacity is not exceeded, and the overflow flag stays clear
    part.ep.capacity_factor = 4.0
    for p in part.parameters():
        p.grad = None
    xs = x_all[sl].clone().requires_grad_()
    ws_ = w_all[sl].clone().requires_grad_()
    out = ep_lib.expert_parallel_forward(part, xs, ws_, idx_all[sl])
    out.backward(dout_all[sl])
    _lib.raise_if_kernel_error()
    part.ep.raise_if_overflow()
    res["out_cap"] = rel(out, ref[sl])
    res["dx_cap"] = rel(xs.grad, xr.grad[sl])
    res["dgate_cap"] = rel(part.gate_proj.grad, full.gate_proj.grad[rank * n:(rank + 1) * n])
    part.ep.capacity_factor = None
    # experts recomputed in backward from the rows that were received (no second exchange): same gradients
    for p in part.parameters():
        p.grad = None
    xs = x_all[sl].clone().requires_grad_()
    ws_ = w_all[sl].clone().requires_grad_()
    out = ep_lib.expert_parallel_forward(part, xs, ws_, idx_all[sl], recompute=True)
    out.backward(dout_all[sl])
    _lib.raise_if_kernel_error()
    res["out_rc"] = rel(out, ref[sl])
    res["dx_rc"] = rel(xs.grad, xr.grad[sl])
    res["dw_rc"] = rel(ws_.grad, wr.grad[sl])
    res["dgate_rc"] = rel(part.gate_proj.grad, full.gate_proj.grad[rank * n:(rank + 1) * n])
    res["ddown_rc"] = rel(part.down_proj.grad, full.down_proj.grad[rank * n:(rank + 1) * n])
    allres = [None] * world
    dist.all_gather_object(allres, res)
    if rank == 0:
        json.dump(allres, open(out_path, "w"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
