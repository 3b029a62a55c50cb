"""Thin launchers for the sm_100a kernels (no autograd here; see `ops/functional.py`).

Each function validates shapes/dtypes, picks strides and calls one `extern "C"`
entry point on the current CUDA stream. Tensors are bf16 unless stated.
"""
from __future__ import annotations

import torch

from .. import _lib

GF_A_MN, GF_B_MN, GF_OUT_F32, GF_ACCUM, GF_BIAS, GF_RESIDUAL, GF_GLU_SILU, GF_GLU_GELU = 1, 2, 4, 8, 16, 32, 64, 128

launch_count = 0  # number of native kernel launches issued through this module


def _count(n: int = 1) -> None:
    global launch_count
    launch_count += n


def _is2d_rowmajor(t: torch.Tensor) -> bool:
    return t.dim() == 2 and t.stride(1) == 1


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16,
         accumulate: bool = False, bias: torch.Tensor | None = None,
         residual: torch.Tensor | None = None, alpha: float = 1.0,
         max_ctas: int = 0) -> torch.Tensor:
    """C = alpha * op(A) @ op(B)^T on the tcgen05 GEMM.

    a: [M,K] (a_mn=False) or [K,M] (a_mn=True); b: [N,K] (b_mn=False) or [K,N] (b_mn=True).
    Row-major 2-D views with unit inner stride; leading strides multiples of 8.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert _is2d_rowmajor(a) and _is2d_rowmajor(b), "operands must be 2-D with unit inner stride"
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        assert not accumulate
    assert out.shape == (M, N) and out.stride(1) == 1
    flags = (GF_A_MN if a_mn else 0) | (GF_B_MN if b_mn else 0)
    if out.dtype == torch.float32:
        flags |= GF_OUT_F32
    else:
        assert out.dtype == torch.bfloat16
    if accumulate:
        flags |= GF_ACCUM
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.numel() == N and bias.is_contiguous()
        flags |= GF_BIAS
    ldr = 0
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (M, N) and residual.stride(1) == 1
        flags |= GF_RESIDUAL
        ldr = residual.stride(0)
    if M == 0 or N == 0:
        return out
    status = _lib.status_buffer(a.device)
    rc = _lib.cuda().tb_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
        flags, _lib.ptr(bias), _lib.ptr(residual), ldr, float(alpha), status.data_ptr(), int(max_ctas),
        _lib.stream_ptr())
    _lib.check(rc, "tb_gemm_bf16")
    _count()
    return out


def gemm_ext(a: torch.Tensor, b: torch.Tensor, a2: torch.Tensor, b2: torch.Tensor, *, b_mn: bool = False,
             out: torch.Tensor | None = None, bias: torch.Tensor | None = None,
             residual: torch.Tensor | None = None) -> torch.Tensor:
    """C = A @ op(B)^T + A2 @ op(B2)^T (+ bias) (+ residual) in ONE launch: the second product (a low-rank adapter
    update) is a few extra k-blocks accumulated into the same TMEM tile.

    a [M, K], a2 [M, r]; b [N, K] and b2 [N, r] (b_mn=False) or b [K, N] and b2 [r, N] (b_mn=True). Problems too small
    for the two-SM kernel run as two GEMMs (the second adds the first as its residual)."""
    assert a.dtype == b.dtype == a2.dtype == b2.dtype == torch.bfloat16
    assert all(_is2d_rowmajor(t) for t in (a, b, a2, b2))
    M, K = a.shape
    N = b.shape[1] if b_mn else b.shape[0]
    r = a2.shape[1]
    assert a2.shape[0] == M and (b2.shape == (r, N) if b_mn else b2.shape == (N, r))
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    assert out.dtype == torch.bfloat16 and out.shape == (M, N) and out.stride(1) == 1
    flags = GF_B_MN if b_mn else 0
    ldr = 0
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.numel() == N and bias.is_contiguous()
        flags |= GF_BIAS
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (M, N) and residual.stride(1) == 1
        flags |= GF_RESIDUAL
        ldr = residual.stride(0)
    if M == 0 or N == 0:
        return out
    rc = 0
    if r % 8 == 0 and a2.stride(0) % 8 == 0 and b2.stride(0) % 8 == 0:
        status = _lib.status_buffer(a.device)
        rc = _lib.cuda().tb_gemm_bf16_ext(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0), flags,
            _lib.ptr(bias), _lib.ptr(residual), ldr, 1.0, a2.data_ptr(), b2.data_ptr(), r, a2.stride(0), b2.stride(0),
            status.data_ptr(), _lib.stream_ptr())
        if rc < 0:
            _lib.check(rc, "tb_gemm_bf16_ext")
    if rc == 1:
        _count()
        return out
    gemm(a, b, b_mn=b_mn, out=out, bias=bias, residual=residual)
    return gemm(a2, b2, b_mn=b_mn, out=out, residual=out)


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float, add_one: bool = False,
                want_rstd: bool = True, out: torch.Tensor | None = None):
    """x: [rows, D] (unit inner stride). Returns (y, rstd[rows] fp32 or None)."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    rows, D = x.shape
    y = out if out is not None else torch.empty((rows, D), dtype=torch.bfloat16, device=x.device)
    rstd = torch.empty((rows,), dtype=torch.float32, device=x.device) if want_rstd else None
    rc = _lib.cuda().tb_rmsnorm_fwd(x.data_ptr(), x.stride(0), w.data_ptr(), y.data_ptr(), y.stride(0),
                                    _lib.ptr(rstd), rows, D, float(eps), 1.0 if add_one else 0.0,
                                    _lib.stream_ptr())
    _lib.check(rc, "tb_rmsnorm_fwd")
    _count()
    return y, rstd


def rmsnorm_bwd(dy, x, w, rstd, add_one: bool = False, want_dw: bool = True,
                dx_accumulate_into: torch.Tensor | None = None):
    """Returns (dx bf16 [rows,D], dw fp32 [D] or None)."""
    rows, D = x.shape
    assert dy.stride(1) == 1 and x.stride(1) == 1
    if dx_accumulate_into is not None:
        dx = dx_accumulate_into
        acc = 1
    else:
        dx = torch.empty((rows, D), dtype=torch.bfloat16, device=x.device)
        acc = 0
    dw = torch.zeros((D,), dtype=torch.float32, device=x.device) if want_dw else None
    rc = _lib.cuda().tb_rmsnorm_bwd(dy.data_ptr(), dy.stride(0), x.data_ptr(), x.stride(0), w.data_ptr(),
                                    rstd.data_ptr(), dx.data_ptr(), dx.stride(0), _lib.ptr(dw), rows, D,
                                    1.0 if add_one else 0.0, acc, _lib.stream_ptr())
    _lib.check(rc, "tb_rmsnorm_bwd")
    _count(2 if want_dw else 1)
    return dx, dw


def rope_(x: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
          backward: bool = False) -> torch.Tensor:
    """In-place half-split RoPE on x [tokens, heads, H] (heads*H contiguous per token).

    positions: int32 [tokens]; cos/sin: fp32 [max_pos, H/2].
    """
    assert x.dtype == torch.bfloat16 and x.dim() == 3 and x.stride(2) == 1 and x.stride(1) == x.shape[2]
    tokens, heads, H = x.shape
    assert positions.dtype == torch.int32 and positions.numel() == tokens and positions.is_contiguous()
    assert cos.dtype == torch.float32 and cos.shape[1] == H // 2 and cos.is_contiguous() and sin.is_contiguous()
    rc = _lib.cuda().tb_rope(x.data_ptr(), x.stride(0), positions.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                             tokens, heads, H, 1 if backward else 0, _lib.stream_ptr())
    _lib.check(rc, "tb_rope")
    _count()
    return x


GLU_SILU, GLU_GELU = 0, 1


def glu_fwd(g: torch.Tensor, u: torch.Tensor, kind: int) -> torch.Tensor:
    rows, Fdim = g.shape
    h = torch.empty((rows, Fdim), dtype=torch.bfloat16, device=g.device)
    rc = _lib.cuda().tb_glu_fwd(g.data_ptr(), g.stride(0), u.data_ptr(), u.stride(0), h.data_ptr(), h.stride(0),
                                rows, Fdim, kind, _lib.stream_ptr())
    _lib.check(rc, "tb_glu_fwd")
    _count()
    return h


def glu_bwd(dh, g, u, kind: int, inplace: bool = False):
    rows, Fdim = g.shape
    dg = g if inplace else torch.empty_like(g)
    du = u if inplace else torch.empty_like(u)
    rc = _lib.cuda().tb_glu_bwd(dh.data_ptr(), dh.stride(0), g.data_ptr(), g.stride(0), u.data_ptr(), u.stride(0),
                                dg.data_ptr(), dg.stride(0), du.data_ptr(), du.stride(0), rows, Fdim, kind,
                                _lib.stream_ptr())
    _lib.check(rc, "tb_glu_bwd")
    _count()
    return dg, du


def embedding_fwd(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    assert ids.dtype == torch.int32 and ids.is_contiguous() and table.dtype == torch.bfloat16
    tokens = ids.numel()
    V, D = table.shape
    out = torch.empty((tokens, D), dtype=torch.bfloat16, device=table.device)
    rc = _lib.cuda().tb_embedding_fwd(ids.data_ptr(), table.data_ptr(), table.stride(0), out.data_ptr(), D,
                                      tokens, D, V, float(scale), _lib.stream_ptr())
    _lib.check(rc, "tb_embedding_fwd")
    _count()
    return out


def embedding_bwd(ids: torch.Tensor, dout: torch.Tensor, dtable: torch.Tensor, scale: float = 1.0) -> None:
    """dtable[ids] += dout * scale (dtable bf16, accumulated in place)."""
    tokens = ids.numel()
    V, D = dtable.shape
    rc = _lib.cuda().tb_embedding_bwd(ids.data_ptr(), dout.data_ptr(), dout.stride(0), dtable.data_ptr(),
                                      dtable.stride(0), tokens, D, V, float(scale), _lib.stream_ptr())
    _lib.check(rc, "tb_embedding_bwd")
    _count()


def logsoftmax_gather(logits: torch.Tensor, targets: torch.Tensor, *, softcap: float = 0.0,
                      temperature: float = 1.0, want_entropy: bool = False):
    """logits fp32 [rows, V]; targets int32 [rows]. Returns (logp, lse, entropy|None), all fp32 [rows]."""
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    rows, V = logits.shape
    logp = torch.empty((rows,), dtype=torch.float32, device=logits.device)
    lse = torch.empty_like(logp)
    ent = torch.empty_like(logp) if want_entropy else None
    rc = _lib.cuda().tb_logsoftmax_gather(logits.data_ptr(), logits.stride(0), targets.data_ptr(), logp.data_ptr(),
                                          lse.data_ptr(), _lib.ptr(ent), rows, V, float(softcap), float(temperature),
                                          _lib.stream_ptr())
    _lib.check(rc, "tb_logsoftmax_gather")
    _count()
    return logp, lse, ent


def dlogits(logits, targets, lse, entropy, dlogp, dent, *, softcap: float = 0.0, temperature: float = 1.0,
            out: torch.Tensor | None = None):
    rows, V = logits.shape
    if out is None:
        out = torch.empty((rows, V), dtype=torch.bfloat16, device=logits.device)
    rc = _lib.cuda().tb_dlogits(logits.data_ptr(), logits.stride(0), _lib.ptr(targets), lse.data_ptr(),
                                _lib.ptr(entropy), _lib.ptr(dlogp), _lib.ptr(dent), out.data_ptr(), out.stride(0),
                                rows, V, float(softcap), float(temperature), _lib.stream_ptr())
    _lib.check(rc, "tb_dlogits")
    _count()
    return out


def sumsq(g: torch.Tensor, out: torch.Tensor) -> None:
    """out[0] += sum(g^2); g flat bf16 or fp32, out fp32 scalar tensor on device."""
    assert g.is_contiguous() and out.dtype == torch.float32
    rc = _lib.cuda().tb_sumsq(g.data_ptr(), g.numel(), 1 if g.dtype == torch.bfloat16 else 0, out.data_ptr(),
                              _lib.stream_ptr())
    _lib.check(rc, "tb_sumsq")
    _count()


def adamw(p32, m, v, g, p16, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0, max_norm=0.0,
          sumsq_buf=None, denom_buf=None) -> None:
    assert p32.dtype == torch.float32 and p32.is_contiguous() and g.is_contiguous()
    n = p32.numel()
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    rc = _lib.cuda().tb_adamw(p32.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(),
                              1 if g.dtype == torch.bfloat16 else 0, _lib.ptr(p16), n, float(lr), float(beta1),
                              float(beta2), float(eps), float(weight_decay), float(bc1), float(bc2),
                              float(grad_scale), float(max_norm), _lib.ptr(sumsq_buf), _lib.ptr(denom_buf),
                              _lib.stream_ptr())
    _lib.check(rc, "tb_adamw")
    _count()


def sgd(p32, mom, g, p16, *, lr, momentum=0.0, weight_decay=0.0, scale=1.0) -> None:
    rc = _lib.cuda().tb_sgd(p32.data_ptr(), _lib.ptr(mom), g.data_ptr(), 1 if g.dtype == torch.bfloat16 else 0,
                            _lib.ptr(p16), p32.numel(), float(lr), float(momentum), float(weight_decay), float(scale),
                            _lib.stream_ptr())
    _lib.check(rc, "tb_sgd")
    _count()


_lib.register_cuda_sigs({
    "tb_attn_fwd": [_lib.P, _lib.P, _lib.P, _lib.P, _lib.P, _lib.I, _lib.I, _lib.I, _lib.I, _lib.I, _lib.I,
                    _lib.LL, _lib.LL, _lib.LL, _lib.LL, _lib.F, _lib.F, _lib.I, _lib.I, _lib.I, _lib.P, _lib.P,
                    _lib.P, _lib.P],
    "tb_attn_delta": [_lib.P, _lib.LL, _lib.P, _lib.LL, _lib.P, _lib.I, _lib.I, _lib.I, _lib.I, _lib.P],
    "tb_attn_bwd": [_lib.P, _lib.P, _lib.P, _lib.P, _lib.P, _lib.P, _lib.P, _lib.P, _lib.P, _lib.I, _lib.I,
                    _lib.I, _lib.I, _lib.I, _lib.I, _lib.LL, _lib.LL, _lib.LL, _lib.LL, _lib.LL, _lib.LL,
                    _lib.F, _lib.F, _lib.I, _lib.I, _lib.I, _lib.P, _lib.P, _lib.P, _lib.P],
})


def _attn_views(q, k, v):
    """q [B,Tq,N,H], k/v [B,Tk,KH,H] with heads*H contiguous per token and tokens evenly strided."""
    B, Tq, N, H = q.shape
    _, Tk, KH, _ = k.shape
    for t in (q, k, v):
        assert t.dtype == torch.bfloat16 and t.stride(3) == 1 and t.stride(2) == H
        assert t.stride(0) == t.shape[1] * t.stride(1), "batch and time must flatten to one row index"
    return B, Tq, Tk, N, KH, H


def attn_fwd(q, k, v, *, scale: float, causal: bool = True, window: int = 0, softcap: float = 0.0,
             q_off: int | None = None, seg_q=None, seg_k=None, want_lse: bool = True):
    """Flash attention forward. Returns (o [B,Tq,N,H] bf16, lse [B,N,Tq] fp32 | None)."""
    B, Tq, Tk, N, KH, H = _attn_views(q, k, v)
    if q_off is None:
        q_off = Tk - Tq
    o = torch.empty((B, Tq, N, H), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, N, Tq), dtype=torch.float32, device=q.device) if want_lse else None
    status = _lib.status_buffer(q.device)
    rc = _lib.cuda().tb_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), _lib.ptr(lse), B, Tq, Tk,
                                 N, KH, H, q.stride(1), k.stride(1), v.stride(1), o.stride(1), float(scale),
                                 float(softcap), 1 if causal else 0, int(window), int(q_off), _lib.ptr(seg_q),
                                 _lib.ptr(seg_k), status.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "tb_attn_fwd")
    _count()
    return o, lse


def attn_bwd(dout, q, k, v, o, lse, *, scale: float, causal: bool = True, window: int = 0, softcap: float = 0.0,
             q_off: int | None = None, seg_q=None, seg_k=None):
    """Flash attention backward. Returns (dq, dk, dv) in bf16 with the shapes of q, k, v."""
    B, Tq, Tk, N, KH, H = _attn_views(q, k, v)
    if q_off is None:
        q_off = Tk - Tq
    assert dout.stride(3) == 1 and dout.stride(2) == H and dout.stride(0) == Tq * dout.stride(1)
    delta = torch.empty((B, N, Tq), dtype=torch.float32, device=q.device)
    lib = _lib.cuda()
    rc = lib.tb_attn_delta(o.data_ptr(), o.stride(1), dout.data_ptr(), dout.stride(1), delta.data_ptr(), B, Tq, N, H,
                           _lib.stream_ptr())
    _lib.check(rc, "tb_attn_delta")
    dq32 = torch.zeros((B, Tq, N, H), dtype=torch.float32, device=q.device)
    dk = torch.empty((B, Tk, KH, H), dtype=torch.bfloat16, device=q.device)
    dv = torch.empty((B, Tk, KH, H), dtype=torch.bfloat16, device=q.device)
    status = _lib.status_buffer(q.device)
    rc = lib.tb_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), dout.data_ptr(), lse.data_ptr(), delta.data_ptr(),
                         dq32.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, Tq, Tk, N, KH, H, q.stride(1), k.stride(1),
                         v.stride(1), dout.stride(1), dk.stride(1), dv.stride(1), float(scale), float(softcap),
                         1 if causal else 0, int(window), int(q_off), _lib.ptr(seg_q), _lib.ptr(seg_k),
                         status.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "tb_attn_bwd")
    dq = torch.empty((B, Tq, N, H), dtype=torch.bfloat16, device=q.device)
    rc = lib.tb_cast_f32_bf16(dq32.data_ptr(), dq.data_ptr(), dq32.numel(), 1.0, _lib.stream_ptr())
    _lib.check(rc, "tb_cast_f32_bf16")
    _count(4)
    return dq, dk, dv


_lib.register_cuda_sigs({
    "tb_kv_write": [_lib.P, _lib.P, _lib.LL, _lib.P, _lib.P, _lib.P, _lib.I, _lib.I, _lib.P, _lib.P, _lib.I, _lib.I, _lib.P],
    "tb_paged_decode": [_lib.P, _lib.LL, _lib.P, _lib.P, _lib.P, _lib.I, _lib.I, _lib.P, _lib.P, _lib.I, _lib.I, _lib.I,
                        _lib.I, _lib.I, _lib.F, _lib.F, _lib.I, _lib.I, _lib.LL, _lib.P, _lib.P, _lib.P, _lib.LL, _lib.P, _lib.P],
    "tb_qkv_post": [_lib.P, _lib.LL, _lib.P, _lib.P, _lib.P, _lib.P, _lib.F, _lib.F, _lib.P, _lib.P, _lib.P, _lib.I,
                    _lib.I, _lib.P, _lib.P, _lib.I, _lib.I, _lib.I, _lib.I, _lib.P],
    "tb_decode_advance": [_lib.P, _lib.P, _lib.P, _lib.P, _lib.P, _lib.LL, _lib.P, _lib.P, _lib.P, _lib.I, _lib.LL, _lib.P,
                          _lib.P, _lib.P, _lib.P, _lib.I, _lib.P],
})


def decode_advance(st: dict, pad_id: int) -> None:
    """The continuous-batching loop's bookkeeping after a sampled token, one kernel for all slots (csrc/decode.cu,
    decode_advance_kernel): append token and log-prob at each live slot's cursor, mark slots that hit an
    end-of-sequence id or their limit, set up the next step's token / position / length, advance the step counter.
    `st`: the engine's static decode buffers."""
    B = st["tokens"].shape[0]
    rc = _lib.cuda().tb_decode_advance(st["next"].data_ptr(), st["next_lp"].data_ptr(), st["done"].data_ptr(),
                                       st["out_tokens"].data_ptr(), st["out_lp"].data_ptr(), st["out_tokens"].stride(0),
                                       st["out_pos"].data_ptr(), st["limit"].data_ptr(), st["eos"].data_ptr(),
                                       st["eos"].numel(), int(pad_id), st["tokens"].data_ptr(), st["positions"].data_ptr(),
                                       st["seq_lens"].data_ptr(), st["step"].data_ptr(), B, _lib.stream_ptr())
    _lib.check(rc, "tb_decode_advance")
    _count()


DECODE_SPLIT_TOKENS = 512


def kv_write(k_new, v_new, seq_ids, positions, page_table, page_size: int, k_pool, v_pool) -> None:
    """Scatter rows k_new / v_new [n_tok, KH*H] into the paged pools [num_pages, page_size, KH*H].

    seq_ids / positions int32 [n_tok] (position < 0 = padding, skipped); page_table int32 [slots, max_pages]."""
    n_tok, row = k_new.shape
    rc = _lib.cuda().tb_kv_write(k_new.data_ptr(), v_new.data_ptr(), k_new.stride(0), seq_ids.data_ptr(),
                                 positions.data_ptr(), page_table.data_ptr(), page_table.shape[1], page_size,
                                 k_pool.data_ptr(), v_pool.data_ptr(), n_tok, row, _lib.stream_ptr())
    _lib.check(rc, "tb_kv_write")
    _count()


def qkv_post(qkv, seq_ids, positions, q_norm_w, k_norm_w, eps: float, add_one: bool, cos, sin, page_table,
             page_size: int, k_pool, v_pool, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """Fused epilogue of the decode-step q/k/v projection: per-head RMS norm of q and k (weights None = no norm),
    RoPE of q and k, q rewritten in place in `qkv` [n_tok, (N + 2 KH) * H], k and v rows written to their pages."""
    n_tok = qkv.shape[0]
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim
    assert cos.dtype == torch.float32 and cos.shape[1] == head_dim // 2 and positions.dtype == torch.int32
    rc = _lib.cuda().tb_qkv_post(qkv.data_ptr(), qkv.stride(0), seq_ids.data_ptr(), positions.data_ptr(),
                                 _lib.ptr(q_norm_w), _lib.ptr(k_norm_w), float(eps), 1.0 if add_one else 0.0,
                                 cos.data_ptr(), sin.data_ptr(), page_table.data_ptr(), page_table.shape[1], page_size,
                                 k_pool.data_ptr(), v_pool.data_ptr(), n_tok, num_heads, num_kv_heads, head_dim,
                                 _lib.stream_ptr())
    _lib.check(rc, "tb_qkv_post")
    _count()


def decode_split_tokens(batch: int, num_kv_heads: int, max_ctx: int = 0) -> int:
    """Context tokens per CTA of `paged_decode` (grid = batch x kv heads x splits). Measured on B200 with 8 kv heads,
    head dim 128, TMA staging: at 64 sequences x 640 tokens 128 / 256 / 512 tokens per CTA take 58 / 56 / 52 us, at
    256 sequences x 768 tokens 512 / 1024 take 161 / 157 us: the per-CTA costs (query load, merge of the warps'
    states, partial write, combine) outweigh a finer balance, so the split is coarse. A context that fits one split
    needs no combine kernel at all (the CTA writes the output row itself)."""
    import os
    forced = os.environ.get("TUNIX_B200_DECODE_SPLIT")
    if forced:
        return int(forced)
    if batch * num_kv_heads >= 512:
        whole = -(-max_ctx // 64) * 64
        return whole if 0 < whole <= 2048 else 1024      # one split per sequence when the context allows
    return DECODE_SPLIT_TOKENS


def paged_decode(q, k_pool, v_pool, page_table, seq_ids, seq_lens, *, num_kv_heads: int, page_size: int, max_ctx: int,
                 scale: float, softcap: float = 0.0, window: int = 0, workspace=None, out=None, split_tokens: int = 0):
    """Single-token attention over a paged KV cache. q [B, N, H] bf16 (row stride free) -> out [B, N, H] bf16.
    `workspace` (two fp32 buffers) must be sized for ceil(max_ctx / split_tokens) splits."""
    B, N, H = q.shape
    assert q.stride(2) == 1 and q.stride(1) == H
    split_tokens = split_tokens or decode_split_tokens(B, num_kv_heads, max_ctx)
    splits = (max_ctx + split_tokens - 1) // split_tokens
    # contiguous pools [pages, page_size, KH * H] can be staged by TMA (one tensor map per pool)
    pool_rows = k_pool.shape[0] * k_pool.shape[1] if (k_pool.is_contiguous() and v_pool.is_contiguous()
                                                      and k_pool.shape == v_pool.shape) else 0
    if workspace is None:
        workspace = (torch.empty(B * N * splits * H, dtype=torch.float32, device=q.device),
                     torch.empty(B * N * splits * 2, dtype=torch.float32, device=q.device))
    if out is None:
        out = torch.empty((B, N, H), dtype=q.dtype, device=q.device)
    rc = _lib.cuda().tb_paged_decode(q.data_ptr(), q.stride(0), k_pool.data_ptr(), v_pool.data_ptr(), page_table.data_ptr(),
                                     page_table.shape[1], page_size, seq_ids.data_ptr(), seq_lens.data_ptr(), B, N,
                                     num_kv_heads, H, max_ctx, float(scale), float(softcap), int(window), int(split_tokens),
                                     pool_rows, workspace[0].data_ptr(), workspace[1].data_ptr(), out.data_ptr(), N * H,
                                     _lib.status_buffer(q.device).data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "tb_paged_decode")
    _count(2)
    return out


# ------------------------------------------------------------------ mixture of experts
_lib.register_cuda_sigs({
    "tb_gemm_grouped_bf16": [_lib.P, _lib.LL, _lib.LL, _lib.LL, _lib.P, _lib.LL, _lib.LL, _lib.LL, _lib.P, _lib.LL, _lib.I,
                             _lib.I, _lib.I, _lib.P, _lib.P, _lib.I, _lib.F, _lib.P, _lib.P],
    "tb_moe_zero_pad": [_lib.P, _lib.LL, _lib.P, _lib.P, _lib.I, _lib.I, _lib.P],
    "tb_moe_scatter_rows": [_lib.P, _lib.LL, _lib.P, _lib.P, _lib.P, _lib.LL, _lib.LL, _lib.I, _lib.I, _lib.P],
    "tb_moe_gather_sum": [_lib.P, _lib.LL, _lib.P, _lib.P, _lib.P, _lib.LL, _lib.P, _lib.LL, _lib.LL, _lib.I, _lib.I, _lib.P],
    "tb_moe_dot_rows": [_lib.P, _lib.LL, _lib.P, _lib.LL, _lib.P, _lib.P, _lib.LL, _lib.I, _lib.I, _lib.P],
    "tb_moe_tiles_rows": [_lib.P, _lib.I, _lib.I, _lib.I, _lib.I, _lib.I, _lib.P, _lib.P, _lib.P],
    "tb_moe_tiles_expert": [_lib.P, _lib.I, _lib.I, _lib.I, _lib.I, _lib.LL, _lib.P, _lib.P, _lib.P],
})

TILE_DESC_BYTES = 32


class TileList:
    """Device-resident tile list of a grouped GEMM: descriptors, their count (device int32) and a host bound."""

    def __init__(self, max_tiles: int, bn: int, device):
        self.desc = torch.empty(max(max_tiles, 1) * TILE_DESC_BYTES, dtype=torch.uint8, device=device)
        self.count = torch.zeros(1, dtype=torch.int32, device=device)
        self.max_tiles, self.bn = max_tiles, bn


def _grouped_bn(n: int) -> int:
    return 256 if n >= 256 else (128 if n >= 128 else 64)


def moe_tiles_rows(seg_off: torch.Tensor, max_rows: int, n_out: int, k_contract: int, b_rows_per_expert: int) -> TileList:
    """Tiles of a GEMM whose output rows are the permuted token rows: [max_rows, n_out] with the contraction
    (k_contract, a multiple of 64) over the feature dimension and B = the stacked expert weights."""
    assert k_contract % 64 == 0
    E = seg_off.numel() - 1
    bn = _grouped_bn(n_out)
    num_n = (n_out + bn - 1) // bn
    tl = TileList((max_rows // 128) * num_n, bn, seg_off.device)
    rc = _lib.cuda().tb_moe_tiles_rows(seg_off.data_ptr(), E, num_n, bn, k_contract // 64, b_rows_per_expert,
                                       tl.desc.data_ptr(), tl.count.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "tb_moe_tiles_rows")
    _count()
    return tl


def moe_tiles_expert(seg_off: torch.Tensor, m_out: int, n_out: int) -> TileList:
    """Tiles of a GEMM with one [m_out, n_out] output per expert, contracted over the expert's row segment."""
    E = seg_off.numel() - 1
    bn = _grouped_bn(n_out)
    tl = TileList(E * ((m_out + 127) // 128) * ((n_out + bn - 1) // bn), bn, seg_off.device)
    rc = _lib.cuda().tb_moe_tiles_expert(seg_off.data_ptr(), E, m_out, n_out, bn, m_out * n_out, tl.desc.data_ptr(),
                                         tl.count.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "tb_moe_tiles_expert")
    _count()
    return tl


def gemm_grouped(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, n_limit: int, tiles: TileList, *,
                 a_mn: bool = False, b_mn: bool = False, accumulate: bool = False) -> torch.Tensor:
    """Grouped GEMM over `tiles`. a, b: 2-D row-major arrays (b = stacked expert matrices viewed 2-D); which
    dimension is contracted follows a_mn / b_mn as in `gemm`. out: bf16 or fp32, 2-D (per-expert outputs are
    addressed through the tile's element offset). n_limit: number of valid output columns per group."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and _is2d_rowmajor(a) and _is2d_rowmajor(b)
    flags = (GF_A_MN if a_mn else 0) | (GF_B_MN if b_mn else 0) | (GF_OUT_F32 if out.dtype == torch.float32 else 0) | \
        (GF_ACCUM if accumulate else 0)
    rc = _lib.cuda().tb_gemm_grouped_bf16(a.data_ptr(), a.shape[0], a.shape[1], a.stride(0), b.data_ptr(), b.shape[0],
                                          b.shape[1], b.stride(0), out.data_ptr(), out.stride(-2), n_limit, flags,
                                          tiles.bn, tiles.desc.data_ptr(), tiles.count.data_ptr(), tiles.max_tiles, 1.0,
                                          _lib.status_buffer().data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "tb_gemm_grouped_bf16")
    _count()
    return out


def moe_zero_pad(buf: torch.Tensor, seg_off: torch.Tensor, counts: torch.Tensor) -> None:
    rc = _lib.cuda().tb_moe_zero_pad(buf.data_ptr(), buf.stride(0), seg_off.data_ptr(), counts.data_ptr(),
                                     counts.numel(), buf.shape[1], _lib.stream_ptr())
    _lib.check(rc, "tb_moe_zero_pad")
    _count()


def moe_scatter_rows(src: torch.Tensor, pos: torch.Tensor, scale, dst: torch.Tensor) -> None:
    """dst[pos[t, j]] = scale[t, j] * src[t] (scale None = 1); pos int32 [T, k], negative = skip."""
    T, k = pos.shape
    rc = _lib.cuda().tb_moe_scatter_rows(src.data_ptr(), src.stride(0), pos.data_ptr(), _lib.ptr(scale), dst.data_ptr(),
                                         dst.stride(0), T, k, src.shape[1], _lib.stream_ptr())
    _lib.check(rc, "tb_moe_scatter_rows")
    _count()


def moe_gather_sum(src: torch.Tensor, pos: torch.Tensor, wts, residual=None) -> torch.Tensor:
    """out[t] = sum_j wts[t, j] * src[pos[t, j]] (+ residual[t]); wts fp32 [T, k] or None."""
    T, k = pos.shape
    D = src.shape[1]
    out = torch.empty((T, D), dtype=torch.bfloat16, device=src.device)
    rc = _lib.cuda().tb_moe_gather_sum(src.data_ptr(), src.stride(0), pos.data_ptr(), _lib.ptr(wts), _lib.ptr(residual),
                                       residual.stride(0) if residual is not None else 0, out.data_ptr(), out.stride(0),
                                       T, k, D, _lib.stream_ptr())
    _lib.check(rc, "tb_moe_gather_sum")
    _count()
    return out


def moe_dot_rows(a: torch.Tensor, b: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    """out[t, j] = <a[t], b[pos[t, j]]> in fp32."""
    T, k = pos.shape
    out = torch.empty((T, k), dtype=torch.float32, device=a.device)
    rc = _lib.cuda().tb_moe_dot_rows(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), pos.data_ptr(), out.data_ptr(),
                                     T, k, a.shape[1], _lib.stream_ptr())
    _lib.check(rc, "tb_moe_dot_rows")
    _count()
    return out


# ------------------------------------------------------------------ GEMMs fused with a collective
_lib.register_cuda_sigs({
    "tb_gemm_ag_bf16": [_lib.P, _lib.I, _lib.I, _lib.I, _lib.LL, _lib.LL, _lib.P, _lib.LL, _lib.P, _lib.LL, _lib.I, _lib.I,
                        _lib.I, _lib.I, _lib.P, _lib.P, _lib.LL, _lib.P, _lib.U, _lib.I, _lib.P, _lib.P],
    "tb_gemm_rs_bf16": [_lib.P, _lib.LL, _lib.P, _lib.LL, _lib.I, _lib.I, _lib.I, _lib.I, _lib.P, _lib.P, _lib.P, _lib.P,
                        _lib.I, _lib.I, _lib.P, _lib.P, _lib.I, _lib.P, _lib.P],
})


def gemm_ag(gathered_ptrs, rank: int, world: int, mode: int, rows: int, cols: int, other: torch.Tensor, out: torch.Tensor,
            M: int, N: int, K: int, ready: torch.Tensor, epoch: int, *, other_mn: bool = False, accumulate: bool = False,
            bias=None, residual=None, n_aux: int = 0) -> torch.Tensor:
    """GEMM whose gathered operand is pulled from the peers inside the kernel (see tb_gemm_ag_bf16 in gemm.cu).

    gathered_ptrs / part_ptrs / done_ptrs below are `SymmBuffer.c_ptrs` pointer tables.
    mode 1: A = gathered [M, K]; mode 2: B = gathered [N, K]; mode 3: B = gathered [K, N] and A = other [K, M]."""
    flags = (GF_OUT_F32 if out.dtype == torch.float32 else 0) | (GF_ACCUM if accumulate else 0)
    if other_mn:
        flags |= GF_B_MN if mode == 1 else GF_A_MN
    if bias is not None:
        flags |= GF_BIAS
    ldr = 0
    if residual is not None:
        flags |= GF_RESIDUAL
        ldr = residual.stride(0)
    rc = _lib.cuda().tb_gemm_ag_bf16(gathered_ptrs, rank, world, mode, rows, cols, other.data_ptr(), other.stride(0), out.data_ptr(),
                                     out.stride(0), M, N, K, flags, _lib.ptr(bias), _lib.ptr(residual), ldr,
                                     ready.data_ptr(), epoch & 0xFFFFFFFF, n_aux, _lib.status_buffer().data_ptr(),
                                     _lib.stream_ptr())
    _lib.check(rc, "tb_gemm_ag_bf16")
    _count()
    return out


def gemm_rs(a: torch.Tensor, b: torch.Tensor, part_ptrs, done_ptrs, out: torch.Tensor, total, work: torch.Tensor,
            rank: int, world: int, M: int, N: int, K: int, *, a_mn: bool = False, b_mn: bool = False, residual=None, n_aux: int = 0) -> torch.Tensor:
    """Row-parallel GEMM with the reduce-scatter of its partial products fused in (tb_gemm_rs_bf16 in gemm.cu).
    `total` is a ctypes.c_uint that carries the counter target of this workspace from call to call."""
    import ctypes
    flags = (GF_A_MN if a_mn else 0) | (GF_B_MN if b_mn else 0)
    assert out.is_contiguous() and (residual is None or residual.is_contiguous())
    rc = _lib.cuda().tb_gemm_rs_bf16(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), M, N, K, flags,
                                     part_ptrs, done_ptrs, out.data_ptr(), _lib.ptr(residual), rank,
                                     world, ctypes.byref(total), work.data_ptr(), n_aux, _lib.status_buffer().data_ptr(),
                                     _lib.stream_ptr())
    _lib.check(rc, "tb_gemm_rs_bf16")
    _count()
    return out


# ------------------------------------------------------------------ expert-parallel row exchange
_lib.register_cuda_sigs({
    "tb_moe_pull_rows": [_lib.P, _lib.I, _lib.LL, _lib.P, _lib.P, _lib.P, _lib.LL, _lib.LL, _lib.I, _lib.P],
    "tb_moe_gather_sum_peer": [_lib.P, _lib.I, _lib.LL, _lib.P, _lib.P, _lib.P, _lib.LL, _lib.P, _lib.LL, _lib.LL, _lib.I,
                               _lib.I, _lib.P],
    "tb_moe_row_scale": [_lib.P, _lib.LL, _lib.P, _lib.P, _lib.LL, _lib.LL, _lib.I, _lib.P],
    "tb_moe_row_dot": [_lib.P, _lib.LL, _lib.P, _lib.LL, _lib.P, _lib.LL, _lib.I, _lib.P],
})


def moe_pull_rows(src_ptrs, world: int, lds: int, src_rank: torch.Tensor, src_row: torch.Tensor, dst: torch.Tensor) -> None:
    """dst[r] = peer[src_rank[r]][src_row[r]] (src_rank < 0: row left as is). src_ptrs: SymmBuffer.c_ptrs."""
    rc = _lib.cuda().tb_moe_pull_rows(src_ptrs, world, lds, src_rank.data_ptr(), src_row.data_ptr(), dst.data_ptr(),
                                      dst.stride(0), src_rank.numel(), dst.shape[1], _lib.stream_ptr())
    _lib.check(rc, "tb_moe_pull_rows")
    _count()


def moe_gather_sum_peer(src_ptrs, world: int, lds: int, dst_rank: torch.Tensor, pos: torch.Tensor, D: int,
                        residual=None) -> torch.Tensor:
    """out[t] = sum_j peer[dst_rank[t, j]][pos[t, j]] (+ residual[t]); dst_rank < 0 skips the slot."""
    T, k = pos.shape
    out = torch.empty((T, D), dtype=torch.bfloat16, device=pos.device)
    rc = _lib.cuda().tb_moe_gather_sum_peer(src_ptrs, world, lds, dst_rank.data_ptr(), pos.data_ptr(), _lib.ptr(residual),
                                            residual.stride(0) if residual is not None else 0, out.data_ptr(),
                                            out.stride(0), T, k, D, _lib.stream_ptr())
    _lib.check(rc, "tb_moe_gather_sum_peer")
    _count()
    return out


def moe_row_scale(src: torch.Tensor, scale: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    out = torch.empty_like(src) if out is None else out
    rc = _lib.cuda().tb_moe_row_scale(src.data_ptr(), src.stride(0), scale.data_ptr(), out.data_ptr(), out.stride(0),
                                      src.shape[0], src.shape[1], _lib.stream_ptr())
    _lib.check(rc, "tb_moe_row_scale")
    _count()
    return out


def moe_row_dot(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    out = torch.empty(a.shape[0], dtype=torch.float32, device=a.device)
    rc = _lib.cuda().tb_moe_row_dot(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), a.shape[0],
                                    a.shape[1], _lib.stream_ptr())
    _lib.check(rc, "tb_moe_row_dot")
    _count()
    return out


# ------------------------------------------------------------------ RL token math
_lib.register_cuda_sigs({
    "tb_policy_loss": [_lib.P, _lib.P, _lib.P, _lib.P, _lib.I, _lib.P, _lib.P, _lib.I, _lib.I, _lib.F, _lib.F, _lib.F, _lib.I,
                       _lib.F, _lib.P, _lib.P, _lib.P, _lib.P, _lib.P, _lib.P],
    "tb_gae_scan": [_lib.P, _lib.P, _lib.P, _lib.I, _lib.I, _lib.F, _lib.F, _lib.P, _lib.P, _lib.P],
})

KL_MODES = {"kl": 0, "mse_kl": 1, "low_var_kl": 2}


def policy_loss(logp, old_logp, ref_logp, adv, mask, is_w, eps_lo: float, eps_hi: float, eps_c, kl_mode: str, kl_clamp):
    """Clipped policy objective and KL per token with their derivatives w.r.t. logp (see csrc/rl_loss.cu).
    Returns (pg, dpg, kl, dkl, flags[2]); kl / dkl are None without a reference."""
    B, T = logp.shape
    f = lambda t: None if t is None else t.detach().float().contiguous()  # noqa: E731
    logp_, old_, ref_, adv_, mask_, isw_ = f(logp), f(old_logp), f(ref_logp), f(adv), f(mask), f(is_w)
    pg, dpg = torch.empty_like(logp_), torch.empty_like(logp_)
    kl = torch.empty_like(logp_) if ref_ is not None else None
    dkl = torch.empty_like(logp_) if ref_ is not None else None
    flags = torch.empty((2, B, T), dtype=torch.float32, device=logp.device)
    rc = _lib.cuda().tb_policy_loss(logp_.data_ptr(), _lib.ptr(old_), _lib.ptr(ref_), adv_.data_ptr(), 1 if adv_.dim() == 2 else 0,
                                    mask_.data_ptr(), _lib.ptr(isw_), B, T, float(eps_lo), float(eps_hi),
                                    float(eps_c) if eps_c else 0.0, KL_MODES[kl_mode], float(kl_clamp) if kl_clamp else 0.0,
                                    pg.data_ptr(), dpg.data_ptr(), _lib.ptr(kl), _lib.ptr(dkl), flags.data_ptr(),
                                    _lib.stream_ptr())
    _lib.check(rc, "tb_policy_loss")
    _count()
    return pg, dpg, kl, dkl, flags


def gae_scan(rewards, values, mask, gamma: float, lam: float):
    """Reverse GAE scan over [B, T] fp32 tensors; returns (advantages before masking, returns)."""
    r, v = rewards.float().contiguous(), values.float().contiguous()
    m = None if mask is None else mask.float().contiguous()
    adv, ret = torch.empty_like(r), torch.empty_like(r)
    rc = _lib.cuda().tb_gae_scan(r.data_ptr(), v.data_ptr(), _lib.ptr(m), r.shape[0], r.shape[1], float(gamma), float(lam),
                                 adv.data_ptr(), ret.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "tb_gae_scan")
    _count()
    return adv, ret


# ------------------------------------------------------------------ fused lm_head -> log-softmax statistics
_lib.register_cuda_sigs({
    "tb_lm_head_lse": [_lib.P, _lib.LL, _lib.P, _lib.LL, _lib.I, _lib.I, _lib.I, _lib.P, _lib.F, _lib.F, _lib.P, _lib.P, _lib.P,
                       _lib.P, _lib.P, _lib.P],
    "tb_lm_head_dlogits": [_lib.P, _lib.LL, _lib.P, _lib.LL, _lib.I, _lib.I, _lib.I, _lib.P, _lib.P, _lib.P, _lib.P, _lib.P,
                           _lib.F, _lib.F, _lib.P, _lib.LL, _lib.P, _lib.P],
})


def lm_head_dlogits(h2: torch.Tensor, w: torch.Tensor, targets, lse, entropy, dlogp, dent, *, softcap: float,
                    temperature: float, out: torch.Tensor) -> bool:
    """out [rows, V] bf16 = gradient with respect to the raw logits h W^T of sum(dlogp * logp + dent * entropy), from
    the epilogue of the GEMM that recomputes the logits (no fp32 logits in memory). Returns False when the problem is
    too small for the two-SM kernel; the caller then recomputes logits into a buffer and runs `dlogits`."""
    import os
    if os.environ.get("TUNIX_B200_NO_FUSED_LSE"):
        return False
    rows, Kd = h2.shape
    V = w.shape[0]
    if rows < 256 or not (_is2d_rowmajor(h2) and _is2d_rowmajor(w)) or h2.stride(0) % 8 or w.stride(0) % 8:
        return False
    assert out.dtype == torch.bfloat16 and out.shape == (rows, V) and out.stride(1) == 1
    rc = _lib.cuda().tb_lm_head_dlogits(h2.data_ptr(), h2.stride(0), w.data_ptr(), w.stride(0), rows, V, Kd,
                                        _lib.ptr(targets), lse.data_ptr(), _lib.ptr(entropy), _lib.ptr(dlogp),
                                        _lib.ptr(dent), 1.0 / float(temperature), float(softcap or 0.0), out.data_ptr(),
                                        out.stride(0), _lib.status_buffer().data_ptr(), _lib.stream_ptr())
    if rc < 0:
        _lib.check(rc, "tb_lm_head_dlogits")
    if rc == 1:
        _count()
    return rc == 1


def lm_head_lse(h2: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, *, softcap: float, temperature: float,
                logp: torch.Tensor, lse: torch.Tensor, entropy) -> bool:
    """log p(target), log-sum-exp and (optionally) entropy of softcap(h W^T) / temperature, written into the given
    fp32 [rows] tensors, without materialising logits (csrc/gemm_2cta.cu). Returns False when the problem is too
    small for the two-SM kernel; the caller then runs its chunked path."""
    import os
    if os.environ.get("TUNIX_B200_NO_FUSED_LSE"):
        return False
    rows, Kd = h2.shape
    V = w.shape[0]
    if rows < 256 or not (_is2d_rowmajor(h2) and _is2d_rowmajor(w)) or h2.stride(0) % 8 or w.stride(0) % 8:
        return False
    num_n = (V + 255) // 256
    partial = torch.empty(rows * num_n * 4, dtype=torch.float32, device=h2.device)
    rc = _lib.cuda().tb_lm_head_lse(h2.data_ptr(), h2.stride(0), w.data_ptr(), w.stride(0), rows, V, Kd, targets.data_ptr(),
                                    1.0 / float(temperature), float(softcap or 0.0), partial.data_ptr(), logp.data_ptr(),
                                    lse.data_ptr(), _lib.ptr(entropy), _lib.status_buffer().data_ptr(), _lib.stream_ptr())
    if rc < 0:
        _lib.check(rc, "tb_lm_head_lse")
    if rc == 1:
        _count(2)
    return rc == 1


# ------------------------------------------------------------------ pre-tiled weights for decode-size GEMMs
_lib.register_cuda_sigs({
    "tb_packed_width": [_lib.I, _lib.I],
    "tb_pack_weight": [_lib.P, _lib.LL, _lib.I, _lib.I, _lib.I, _lib.P, _lib.P],
    "tb_pack_weight_glu": [_lib.P, _lib.LL, _lib.I, _lib.I, _lib.I, _lib.P, _lib.P],
    "tb_gemm_packed_bf16": [_lib.P, _lib.LL, _lib.P, _lib.I, _lib.P, _lib.LL, _lib.I, _lib.I, _lib.I, _lib.I, _lib.P, _lib.P,
                            _lib.LL, _lib.F, _lib.P, _lib.P],
})


class PackedWeight:
    """A K-major weight [N, K] re-tiled for streaming (csrc/gemm.cu, tb_pack_weight): per (n tile of `width` rows,
    64-column k block) one contiguous, pre-swizzled block. `refresh` re-packs after the source changed.

    `glu=True`: the weight is [gate rows; up rows]; the rows are interleaved in groups of 16 = 8 gate + their 8 up
    rows, which lets `gemm_packed(..., glu=kind)` apply the gated activation in its epilogue and write N / 2 columns."""

    def __init__(self, weight: torch.Tensor, width: int | None = None, glu: bool = False):
        assert weight.dtype == torch.bfloat16 and _is2d_rowmajor(weight)
        self.N, self.K = weight.shape
        self.glu = bool(glu)
        assert not glu or self.N % 16 == 0
        self.width = int(width) if width else int(_lib.cuda().tb_packed_width(self.N, self.K))
        nbytes = -(-self.N // self.width) * -(-self.K // 64) * self.width * 128
        self.data = torch.empty(nbytes, dtype=torch.uint8, device=weight.device)
        self.refresh(weight)

    def refresh(self, weight: torch.Tensor) -> None:
        assert weight.shape == (self.N, self.K) and weight.dtype == torch.bfloat16 and _is2d_rowmajor(weight)
        fn = _lib.cuda().tb_pack_weight_glu if self.glu else _lib.cuda().tb_pack_weight
        rc = fn(weight.data_ptr(), weight.stride(0), self.N, self.K, self.width, self.data.data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "tb_pack_weight")
        _count()


def gemm_packed(a: torch.Tensor, pw: PackedWeight, *, out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16,
                accumulate: bool = False, bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
                alpha: float = 1.0, glu: int | None = None) -> torch.Tensor:
    """C = alpha * A @ W^T with W given as a PackedWeight; same epilogue options as `gemm`. `glu` (GLU_SILU / GLU_GELU)
    with a weight packed with `glu=True`: C [M, N / 2] = act(A @ Wgate^T) * (A @ Wup^T), computed in the epilogue."""
    assert a.dtype == torch.bfloat16 and _is2d_rowmajor(a)
    M, K = a.shape
    assert K == pw.K, f"contraction mismatch {K} vs {pw.K}"
    N = pw.N
    if glu is not None:
        assert pw.glu and not accumulate and bias is None and residual is None and alpha == 1.0
        if out is None:
            out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device)
        assert out.shape == (M, N // 2) and out.dtype == torch.bfloat16 and out.stride(1) == 1
        if M == 0:
            return out
        rc = _lib.cuda().tb_gemm_packed_bf16(a.data_ptr(), a.stride(0), pw.data.data_ptr(), pw.width, out.data_ptr(),
                                             out.stride(0), M, N, K, GF_GLU_SILU if glu == GLU_SILU else GF_GLU_GELU, 0, 0, 0, 1.0,
                                             _lib.status_buffer(a.device).data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "tb_gemm_packed_bf16")
        _count()
        return out
    assert not pw.glu, "a weight packed for the gated epilogue needs glu="
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        assert not accumulate
    assert out.shape == (M, N) and out.stride(1) == 1
    flags = 0
    if out.dtype == torch.float32:
        flags |= GF_OUT_F32
    else:
        assert out.dtype == torch.bfloat16
    if accumulate:
        flags |= GF_ACCUM
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.numel() == N and bias.is_contiguous()
        flags |= GF_BIAS
    ldr = 0
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (M, N) and residual.stride(1) == 1
        flags |= GF_RESIDUAL
        ldr = residual.stride(0)
    if M == 0:
        return out
    rc = _lib.cuda().tb_gemm_packed_bf16(a.data_ptr(), a.stride(0), pw.data.data_ptr(), pw.width, out.data_ptr(), out.stride(0),
                                         M, N, K, flags, _lib.ptr(bias), _lib.ptr(residual), ldr, float(alpha),
                                         _lib.status_buffer(a.device).data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "tb_gemm_packed_bf16")
    _count()
    return out
