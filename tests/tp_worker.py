"""Worker of tests/test_tp_gpu.py: launched with torch.distributed.run, one rank per GPU."""
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
    from tunix_b200.parallel import tp as tp_lib
    tp = tp_lib.TPContext(device=dev)
    res = {"fused": tp.fused}
    torch.manual_seed(100 + rank)
    for (M, K, N) in [(1024, 512, 768), (2048, 1024, 256)]:
        m = M // world
        x_s = torch.randn(m, K, device=dev).to(torch.bfloat16)
        torch.manual_seed(7)
        w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)          # same on all ranks
        torch.manual_seed(100 + rank)
        xg_ref = tp.all_gather_rows(x_s)
        for rep in range(2):                                                   # second pass checks the epoch logic
            y, xg = tp.ag_gemm(x_s, w)
            _lib.raise_if_kernel_error()
            res[f"ag_{M}_{rep}"] = rel(y, xg_ref.float() @ w.float().t())
            res[f"ag_copy_{M}_{rep}"] = float((xg.float() - xg_ref.float()).abs().max())
        dy = torch.randn(M, N, device=dev).to(torch.bfloat16)
        g = tp.ag_wgrad(dy, x_s)
        _lib.raise_if_kernel_error()
        res[f"wgrad_{M}"] = rel(g, dy.float().t() @ xg_ref.float())
        acc = torch.ones(N, K, device=dev)
        tp.ag_wgrad(dy, x_s, out=acc, accumulate=True)
        res[f"wgrad_acc_{M}"] = rel(acc, dy.float().t() @ xg_ref.float() + 1)
        # row parallel: every rank holds different x / w slices; result = reduce-scatter of the products
        xr = torch.randn(M, K, device=dev).to(torch.bfloat16)
        wr = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
        res_s = torch.randn(m, N, device=dev).to(torch.bfloat16)
        full = (xr.float() @ wr.float().t())
        dist.all_reduce(full)
        for rep in range(2):
            ys = tp.gemm_rs(xr, wr, residual_s=res_s)
            _lib.raise_if_kernel_error()
            res[f"rs_{M}_{rep}"] = rel(ys, full[rank * m:(rank + 1) * m] + res_s.float())
    # ---- a sliced model against the whole one
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    # heads and kv heads must divide by the number of ranks (4 / 2 for the 2-rank test, more for larger groups)
    cfg = ModelConfig(family="llama3", num_layers=2, vocab_size=512, embed_dim=256, hidden_dim=512 * max(world // 4, 1),
                      num_heads=max(4, world), head_dim=64, num_kv_heads=max(2, world), dtype=torch.bfloat16, max_position=256)
    whole = create_model(cfg, device=dev, seed=0)
    sliced = create_model(cfg, device=dev, seed=0)
    tp_lib.apply_tensor_parallel(sliced, tp)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, 512, (2 * world, 128), generator=g).to(dev)

    def loss_of(model):
        hidden, _ = model(toks, skip_lm_head=True)
        logp, _ = model.token_logprobs(hidden[:, :-1], tp_lib.local_batch(model, toks)[:, 1:])
        return -logp.sum()
    l_whole = loss_of(whole)
    l_whole.backward()
    l_sl = loss_of(sliced)
    l_sl.backward()
    _lib.raise_if_kernel_error()
    tot = l_sl.detach().clone()
    dist.all_reduce(tot)
    tp_lib.allreduce_replicated_grads(sliced, tp)
    res["model_loss_rel"] = abs(float(tot) - float(l_whole)) / abs(float(l_whole))
    gw = whole.layers[0].mlp.down_proj.weight.grad
    n = gw.shape[1] // world
    res["model_grad_row"] = rel(sliced.layers[0].mlp.down_proj.weight.grad, gw[:, rank * n:(rank + 1) * n])
    gq = whole.layers[1].self_attn.q_proj.weight.grad
    n = gq.shape[0] // world
    res["model_grad_col"] = rel(sliced.layers[1].self_attn.q_proj.weight.grad, gq[rank * n:(rank + 1) * n])
    res["model_grad_embed"] = rel(sliced.embed_tokens.grad, whole.embed_tokens.grad)
    # ---- timing at a training shape: fused all-gather + GEMM against NCCL all-gather followed by the GEMM
    if len(sys.argv) > 2 and sys.argv[2] == "bench":
        from tunix_b200.ops import kernels as K
        M, Kd, N = 16384, 4096, 14336 // world
        x_s = torch.randn(M // world, Kd, device=dev).to(torch.bfloat16)
        w = (torch.randn(N, Kd, device=dev) * 0.02).to(torch.bfloat16)

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
        res["bench_ag_fused_ms"] = timed(lambda: tp.ag_gemm(x_s, w))
        res["bench_ag_nccl_ms"] = timed(lambda: K.gemm(tp.all_gather_rows(x_s), w))
        res["bench_gemm_only_ms"] = timed(lambda: K.gemm(xg_full, w)) if (xg_full := tp.all_gather_rows(x_s)) is not None else 0
        xr = torch.randn(M, Kd // world * 2, device=dev).to(torch.bfloat16)
        wr = (torch.randn(4096, Kd // world * 2, device=dev) * 0.02).to(torch.bfloat16)
        res["bench_rs_fused_ms"] = timed(lambda: tp.gemm_rs(xr, wr))
        res["bench_rs_nccl_ms"] = timed(lambda: tp.reduce_scatter_rows(K.gemm(xr, wr)))
        _lib.raise_if_kernel_error()
    allres = [None] * world
    dist.all_gather_object(allres, res)
    if rank == 0:
        json.dump(allres, open(out_path, "w"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
