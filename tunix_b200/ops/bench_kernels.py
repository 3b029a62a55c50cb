"""Kernel micro-benchmarks: `python -m tunix_b200.ops.bench_kernels <kernel> [--shape flags]`.

Each run does warm-up launches, then times `--iters` launches with CUDA events on the launching stream,
flushing L2 (a 256 MiB memset) between iterations, and prints one JSON line with the median time, the
achieved TFLOP/s or GB/s and its fraction of the measured peak (MEASURED_PEAKS.json at the repository
root when present, else the fallback 1590 TFLOP/s / 6650 GB/s). The same entry point is what the ncu
captures in `profiles/` run (small shapes, few iterations).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


def _time(fn, iters: int, warmup: int = 3, flush: bool = True):
    for _ in range(warmup):
        fn()
    buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    times = []
    for _ in range(iters):
        if buf is not None:
            buf.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "attn_fwd", "attn_bwd", "rmsnorm", "adamw", "logsoftmax", "sample",
                                       "glu", "moe", "paged_decode", "lm_head", "lm_head_bwd", "lora"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--a-mn", action="store_true")
    ap.add_argument("--b-mn", action="store_true")
    ap.add_argument("--split", type=int, default=0, help="paged_decode: context tokens per CTA (0 = chosen from the batch)")
    ap.add_argument("--max-ctx", type=int, default=0, help="paged_decode: size the grid for this context (0 = --seq)")
    ap.add_argument("--packed", action="store_true", help="gemm: B as a pre-tiled PackedWeight (decode-size M)")
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--numel", type=int, default=1 << 28)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--ffn", type=int, default=768)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)
    from tunix_b200 import _lib
    from tunix_b200.ops import kernels as K
    peak_tf, peak_gb, src = _peaks()
    dev = "cuda"
    bf = torch.bfloat16
    out = {"kernel": args.kernel, "peaks": src}
    if args.kernel == "gemm":
        M, N, Kd = args.m, args.n, args.k
        A = torch.randn((Kd, M) if args.a_mn else (M, Kd), device=dev, dtype=bf)
        B = torch.randn((Kd, N) if args.b_mn else (N, Kd), device=dev, dtype=bf)
        C = torch.empty(M, N, device=dev, dtype=bf)
        if args.packed:
            pw = K.PackedWeight(B)
            ms = _time(lambda: K.gemm_packed(A, pw, out=C), args.iters, args.warmup)
            out.update(packed_width=pw.width)
        else:
            ms = _time(lambda: K.gemm(A, B, a_mn=args.a_mn, b_mn=args.b_mn, out=C), args.iters, args.warmup)
        tf = 2.0 * M * N * Kd / ms / 1e9
        gb = (M * Kd + N * Kd + M * N) * 2 / ms / 1e6
        out.update(shape=[M, N, Kd], ms=ms, tflops=tf, frac_of_peak=tf / peak_tf, gbs=gb, frac_of_copy_bw=gb / peak_gb)
    elif args.kernel in ("attn_fwd", "attn_bwd"):
        B_, T, N, KH, H = args.batch, args.seq, args.heads, args.kv_heads, args.head_dim
        q = torch.randn(B_, T, N, H, device=dev, dtype=bf)
        k = torch.randn(B_, T, KH, H, device=dev, dtype=bf)
        v = torch.randn_like(k)
        sc = 1.0 / math.sqrt(H)
        fl = 4.0 * B_ * N * T * T * H / 2
        if args.kernel == "attn_fwd":
            ms = _time(lambda: K.attn_fwd(q, k, v, scale=sc), args.iters, args.warmup)
        else:
            o, lse = K.attn_fwd(q, k, v, scale=sc)
            do = torch.randn_like(q)
            ms = _time(lambda: K.attn_bwd(do, q, k, v, o, lse, scale=sc), args.iters, args.warmup)
            fl *= 2.5
        tf = fl / ms / 1e9
        out.update(shape=[B_, T, N, KH, H], ms=ms, tflops=tf, frac_of_peak=tf / peak_tf)
    elif args.kernel == "rmsnorm":
        x = torch.randn(args.rows, args.dim, device=dev, dtype=bf)
        w = torch.ones(args.dim, device=dev, dtype=bf)
        ms = _time(lambda: K.rmsnorm_fwd(x, w, 1e-6), args.iters, args.warmup)
        gb = 2.0 * x.numel() * 2 / ms / 1e6
        out.update(shape=[args.rows, args.dim], ms=ms, gbs=gb, frac_of_peak=gb / peak_gb)
    elif args.kernel == "glu":
        g = torch.randn(args.rows, args.dim, device=dev, dtype=bf)
        u = torch.randn_like(g)
        ms = _time(lambda: K.glu_fwd(g, u, 0), args.iters, args.warmup)
        gb = 3.0 * g.numel() * 2 / ms / 1e6
        out.update(shape=[args.rows, args.dim], ms=ms, gbs=gb, frac_of_peak=gb / peak_gb)
    elif args.kernel == "adamw":
        n = args.numel
        p32, m, v = (torch.zeros(n, device=dev) for _ in range(3))
        g = torch.randn(n, device=dev, dtype=bf)
        p16 = torch.empty(n, device=dev, dtype=bf)
        ss = torch.ones(1, device=dev)
        ms = _time(lambda: K.adamw(p32, m, v, g, p16, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, step=3,
                                   max_norm=1.0, sumsq_buf=ss), args.iters, args.warmup, flush=False)
        gb = n * (3 * 4 * 2 + 2 + 2) / ms / 1e6
        out.update(numel=n, ms=ms, gbs=gb, frac_of_peak=gb / peak_gb)
    elif args.kernel == "logsoftmax":
        z = torch.randn(args.rows, args.vocab, device=dev)
        tg = torch.randint(0, args.vocab, (args.rows,), device=dev, dtype=torch.int32)
        ms = _time(lambda: K.logsoftmax_gather(z, tg), args.iters, args.warmup)
        gb = z.numel() * 4 / ms / 1e6
        out.update(shape=[args.rows, args.vocab], ms=ms, gbs=gb, frac_of_peak=gb / peak_gb)
    elif args.kernel == "sample":
        from tunix_b200.ops import sampling_kernels as S
        z = torch.randn(args.rows, args.vocab, device=dev)
        ms = _time(lambda: S.sample(z, 1.0, None, None, 1, 0, want_logprob=True), args.iters, args.warmup)
        gb = 3.0 * z.numel() * 4 / ms / 1e6
        out.update(shape=[args.rows, args.vocab], ms=ms, gbs_3pass=gb, frac_of_peak=gb / peak_gb)
    elif args.kernel == "lm_head":
        from tunix_b200.ops import functional as F
        rows, V, D = args.rows, args.vocab, args.dim
        h = (torch.randn(rows, D, device=dev) * 0.5).to(bf)
        w = (torch.randn(V, D, device=dev) * 0.02).to(bf)
        tg = torch.randint(0, V, (rows,), device=dev)
        with torch.no_grad():
            ms = _time(lambda: F.lm_head_logprobs(h, w, tg, chunk=4096), args.iters, args.warmup)
        tf = 2.0 * rows * V * D / ms / 1e9
        out.update(shape=[rows, V, D], ms=ms, tflops=tf, frac_of_peak=tf / peak_tf,
                   fused=not bool(os.environ.get("TUNIX_B200_NO_FUSED_LSE")))
    elif args.kernel == "lm_head_bwd":
        # forward + backward of the fused log-prob head; TUNIX_B200_NO_FUSED_LSE=1 gives the path with fp32 logits buffers
        from tunix_b200.ops import functional as F
        rows, V, D = args.rows, args.vocab, args.dim
        h = (torch.randn(rows, D, device=dev) * 0.5).to(bf).requires_grad_()
        w = (torch.randn(V, D, device=dev) * 0.02).to(bf).requires_grad_()
        tg = torch.randint(0, V, (rows,), device=dev)

        def step():
            h.grad = w.grad = None
            lp, _ = F.lm_head_logprobs(h, w, tg, chunk=2048)
            lp.sum().backward()
        ms = _time(step, args.iters, args.warmup)
        tf = 4 * 2.0 * rows * V * D / ms / 1e9          # forward GEMM + recompute + dh + dW
        out.update(shape=[rows, V, D], ms=ms, tflops=tf, frac_of_peak=tf / peak_tf,
                   fused=not bool(os.environ.get("TUNIX_B200_NO_FUSED_LSE")))
    elif args.kernel == "lora":
        # LoRA projection forward + backward: adapter carried by the base GEMM against base GEMM + two low-rank GEMMs
        from tunix_b200.ops import functional as F
        M, N, Kd, r = args.m, args.n, args.k, 16
        x = (torch.randn(M, Kd, device=dev) * 0.5).to(bf).requires_grad_()
        w = (torch.randn(N, Kd, device=dev) * 0.02).to(bf)
        a = (torch.randn(r, Kd, device=dev) * 0.02).to(bf).requires_grad_()
        b = (torch.randn(N, r, device=dev) * 0.02).to(bf).requires_grad_()
        g = torch.randn(M, N, device=dev).to(bf)

        def fused():
            x.grad = a.grad = b.grad = None
            F.lora_linear(x, w, None, a, b, 2.0).backward(g)

        def unfused():
            x.grad = a.grad = b.grad = None
            F.lora_delta(x, a, b, F.linear(x, w), 2.0).backward(g)
        ms_f, ms_u = _time(fused, args.iters, args.warmup), _time(unfused, args.iters, args.warmup)
        tf = 2 * 2.0 * M * N * Kd / ms_f / 1e9
        out.update(shape=[M, N, Kd, r], ms=ms_f, ms_unfused=ms_u, tflops=tf, frac_of_peak=tf / peak_tf)
    elif args.kernel == "paged_decode":
        Bn, ctx, N, KH, H, page = args.batch, args.seq, args.heads, args.kv_heads, args.head_dim, 64
        max_pages = (ctx + page - 1) // page
        kp = torch.randn(Bn * max_pages, page, KH * H, device=dev, dtype=bf)
        vp = torch.randn_like(kp)
        table = torch.randperm(Bn * max_pages, device=dev).int().view(Bn, max_pages)
        lens = torch.full((Bn,), ctx, device=dev, dtype=torch.int32)
        slots = torch.arange(Bn, device=dev, dtype=torch.int32)
        q = torch.randn(Bn, N, H, device=dev, dtype=bf)
        ms = _time(lambda: K.paged_decode(q, kp, vp, table, slots, lens, num_kv_heads=KH, page_size=page,
                                          max_ctx=args.max_ctx or ctx, scale=1.0 / math.sqrt(H), split_tokens=args.split),
                   args.iters, args.warmup)
        gb = 2.0 * Bn * ctx * KH * H * 2 / ms / 1e6
        out.update(shape=[Bn, ctx, N, KH, H], ms=ms, gbs=gb, frac_of_peak=gb / peak_gb,
                   split_tokens=args.split or K.decode_split_tokens(Bn, KH, args.max_ctx or ctx))
    elif args.kernel == "moe":
        from tunix_b200.ops import moe
        T, E, k, D, Fd = args.rows, args.experts, args.topk, args.dim, args.ffn
        x = (torch.randn(T, D, device=dev) * 0.5).to(bf).requires_grad_()
        ws = [(torch.randn(E, Fd, D, device=dev) * 0.02).to(bf).requires_grad_() for _ in range(2)]
        ws.append((torch.randn(E, D, Fd, device=dev) * 0.02).to(bf).requires_grad_())
        for w in ws:
            w.main_grad = torch.zeros(w.shape, dtype=torch.float32, device=dev)
        wt, idx = torch.topk(torch.softmax(torch.randn(T, E, device=dev), -1), k, -1)
        dout = torch.randn(T, D, device=dev).to(bf)
        ms_f = _time(lambda: moe.experts(x, wt, idx, *ws), args.iters, args.warmup)

        def fb():
            moe.experts(x, wt, idx, *ws).backward(dout)
        ms = _time(fb, args.iters, args.warmup)
        fl_f = 2.0 * T * k * D * Fd * 3
        out.update(shape=[T, E, k, D, Fd], fwd_ms=ms_f, fwd_bwd_ms=ms, fwd_tflops=fl_f / ms_f / 1e9,
                   fwd_bwd_tflops=3 * fl_f / ms / 1e9, frac_of_peak=3 * fl_f / ms / 1e9 / peak_tf)
    _lib.raise_if_kernel_error()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
