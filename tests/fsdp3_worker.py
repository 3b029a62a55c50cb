"""Worker of tests/test_fsdp3_gpu.py: launched with torch.distributed.run, one rank per GPU."""
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
    from tunix_b200.parallel import fsdp3
    comm = fsdp3.CommContext(device=dev)
    res = {"fused": comm.fused}
    for (M, K, N) in [(512, 512, 1024), (1000, 1024, 2048)]:
        torch.manual_seed(50 + rank)
        n = N // world
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)                   # this rank's tokens
        w_s = (torch.randn(n, K, device=dev) * 0.05).to(torch.bfloat16)         # this rank's rows of W
        bias = torch.randn(N, device=dev).to(torch.bfloat16)
        resid = torch.randn(M, N, device=dev).to(torch.bfloat16)
        w_full = comm.all_gather_rows(w_s)
        for rep in range(3):                                                    # alternating staging buffers
            y = comm.gemm_gather_w(x, w_s, bias, resid)
            _lib.raise_if_kernel_error()
            res[f"fwd_{M}_{rep}"] = rel(y, x.float() @ w_full.float().t() + bias.float() + resid.float())
        dy = torch.randn(M, N, device=dev).to(torch.bfloat16)
        dx = comm.gemm_gather_w_t(dy, w_s)
        _lib.raise_if_kernel_error()
        res[f"dgrad_{M}"] = rel(dx, dy.float() @ w_full.float())
        if M % 8 == 0:
            g = comm.wgrad_scatter(dy, x)
            _lib.raise_if_kernel_error()
            full = dy.float().t() @ x.float()
            dist.all_reduce(full)
            res[f"wgrad_{M}"] = rel(g, full[rank * n:(rank + 1) * n])
    # ---- sharded model against the whole one: same loss, gradients = the whole model's rows (summed over ranks)
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    cfg = ModelConfig(family="llama3", num_layers=2, vocab_size=512, embed_dim=256, hidden_dim=512, num_heads=4, head_dim=64,
                      num_kv_heads=2, dtype=torch.bfloat16, max_position=256)
    whole = create_model(cfg, device=dev, seed=0)
    sharded = create_model(cfg, device=dev, seed=0)
    fsdp3.apply_weight_sharding(sharded, comm)
    g = torch.Generator().manual_seed(3)
    toks_all = torch.randint(0, 512, (2 * world, 128), generator=g).to(dev)
    toks = toks_all[2 * rank:2 * rank + 2]

    def loss_of(model, t):
        hidden, _ = model(t, skip_lm_head=True)
        logp, _ = model.token_logprobs(hidden[:, :-1], t[:, 1:])
        return -logp.sum()
    lw = loss_of(whole, toks_all)
    lw.backward()
    ls = loss_of(sharded, toks)
    ls.backward()
    _lib.raise_if_kernel_error()
    tot = ls.detach().clone()
    dist.all_reduce(tot)
    fsdp3.sync_replicated_grads(sharded, comm)
    res["model_loss_rel"] = abs(float(tot) - float(lw)) / abs(float(lw))
    gw = whole.layers[0].mlp.down_proj.weight.grad
    n = gw.shape[0] // world
    res["model_grad_sharded"] = rel(sharded.layers[0].mlp.down_proj.weight.grad, gw[rank * n:(rank + 1) * n])
    res["model_grad_embed"] = rel(sharded.embed_tokens.grad, whole.embed_tokens.grad)
    if len(sys.argv) > 2 and sys.argv[2] == "bench":
        from tunix_b200.ops import kernels as K

        def timed(fn, iters=10):
            for _ in range(3):
                fn()
            dist.barrier()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(iters):
                fn()
            e.record()
            torch.cuda.synchronize()
            t = torch.tensor([s.elapsed_time(e) / iters], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t)
        M = 16384
        for name, (N, Kd) in {"gate": (14336, 4096), "down": (4096, 14336), "q": (4096, 4096)}.items():
            x = torch.randn(M, Kd, device=dev).to(torch.bfloat16)
            w_s = (torch.randn(N // world, Kd, device=dev) * 0.02).to(torch.bfloat16)
            w_full = comm.all_gather_rows(w_s)
            res[f"bench_{name}_fused_ms"] = timed(lambda: comm.gemm_gather_w(x, w_s))
            res[f"bench_{name}_nccl_ms"] = timed(lambda: K.gemm(x, comm.all_gather_rows(w_s)))
            res[f"bench_{name}_gemm_ms"] = timed(lambda: K.gemm(x, w_full))
        _lib.raise_if_kernel_error()
    allres = [None] * world
    dist.all_gather_object(allres, res)
    if rank == 0:
        json.dump(allres, open(out_path, "w"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
