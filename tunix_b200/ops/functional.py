"""Differentiable ops used by the models.

Each op has two implementations with the same signature:
  * CUDA bf16 tensors -> hand-written sm_100a kernels (`ops/kernels.py`) wrapped in
    `torch.autograd.Function`s with hand-derived backward passes;
  * anything else (CPU, fp32) -> the PyTorch reference in `ops/reference.py`.
On a CUDA device the native library is mandatory: a missing build raises instead of
quietly running the reference.

Weight gradients can be written straight into a preallocated flat buffer: if a
parameter carries a `main_grad` tensor (fp32 or bf16, same shape), the wgrad GEMM
accumulates into it in its epilogue and autograd sees no gradient for that parameter.
"""
from __future__ import annotations

import contextlib

import torch

from . import kernels as K
from . import reference as R


_library_mode = False


@contextlib.contextmanager
def library_ops():
    """Route every op of this module through stock PyTorch (cuBLAS GEMMs, the library's fused attention, unfused
    element-wise ops) instead of this package's kernels, on any device. This is the in-repo baseline that
    benchmarks measure the kernels against; nothing else uses it."""
    global _library_mode
    prev, _library_mode = _library_mode, True
    try:
        yield
    finally:
        _library_mode = prev


def _native(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and not _library_mode


def _deliver_grad(param, g: torch.Tensor):
    """Hand a parameter gradient to its owner: added into `param.main_grad` when the optimizer gave the parameter a
    slot in its flat gradient buffer (then autograd sees None), returned for autograd otherwise. Optimizers that
    reduce a layer's gradients while backward is still running rely on every gradient of the layer having arrived
    this way by the time backward leaves the layer."""
    mg = getattr(param, "main_grad", None)
    if mg is None:
        return g
    mg.add_(g.reshape(mg.shape).to(mg.dtype))
    param.grad_added_to_main_grad = True
    return None


def _flat2d(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    return x2


# ----------------------------------------------------------------------------- linear
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, residual):
        x2 = _flat2d(x)
        r2 = _flat2d(residual) if residual is not None else None
        # The output is allocated with its final shape (not a view made inside this Function), so
        # a consumer such as the in-place RoPE may overwrite it.
        y = torch.empty((*x.shape[:-1], w.shape[0]), dtype=torch.bfloat16, device=x.device)
        K.gemm(x2, w, bias=bias, residual=r2, out=y.view(-1, w.shape[0]))
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.x_shape = x.shape
        ctx.w_ref = w
        ctx.b_ref = bias
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _flat2d(dy)
        dx = dw = db = dres = None
        if ctx.needs_input_grad[0]:
            dx = K.gemm(dy2, w, b_mn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:
                K.gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, accumulate=True)
                ctx.w_ref.grad_added_to_main_grad = True
            else:
                dw = K.gemm(dy2, x2, a_mn=True, b_mn=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _deliver_grad(ctx.b_ref, dy2.float().sum(0).to(dy.dtype))
        if ctx.has_res and ctx.needs_input_grad[3]:
            dres = dy
        return dx, dw, db, dres


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
           residual: torch.Tensor | None = None) -> torch.Tensor:
    """y = x @ w^T (+ bias) (+ residual); w is [out, in] as in HF checkpoints."""
    if _native(x) and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _LinearFn.apply(x, w, bias, residual)
    y = torch.nn.functional.linear(x, w.to(x.dtype), None if bias is None else bias.to(x.dtype))
    return y if residual is None else y + residual


class _LoraDeltaFn(torch.autograd.Function):
    """y = base + scale * (x A^T) B^T with A [r, in], B [out, r]."""

    @staticmethod
    def forward(ctx, x, a, b, base, scale):
        x2 = _flat2d(x)
        t = K.gemm(x2, a)                                   # [M, r]
        # allocated with its final shape: a consumer (the in-place RoPE) may overwrite the output, which autograd
        # forbids for a view made inside this Function
        y = torch.empty(base.shape, dtype=torch.bfloat16, device=x.device)
        K.gemm(t, b, residual=_flat2d(base), alpha=scale, out=y.view(-1, base.shape[-1]))
        ctx.save_for_backward(x2, a, b, t)
        ctx.scale = scale
        ctx.x_shape = x.shape
        ctx.a_ref, ctx.b_ref = a, b
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, a, b, t = ctx.saved_tensors
        dy2 = _flat2d(dy)
        s = ctx.scale
        dt = K.gemm(dy2, b, b_mn=True, alpha=s)              # [M, r] = s * dy B
        db = K.gemm(dy2, t, a_mn=True, b_mn=True, alpha=s)   # [out, r]
        da = K.gemm(dt, x2, a_mn=True, b_mn=True)            # [r, in]
        dx = None
        if ctx.needs_input_grad[0]:
            dx = K.gemm(dt, a, b_mn=True).view(ctx.x_shape)
        return dx, _deliver_grad(ctx.a_ref, da), _deliver_grad(ctx.b_ref, db), dy, None


class _LoraLinearFn(torch.autograd.Function):
    """y = x W^T + scale * (x A^T) B^T (+ bias) (+ residual) with the adapter product carried by the base GEMM: the
    rank-r intermediate t = scale * x A^T is a second contraction segment of the same launch (forward) and so is
    dt = scale * dy B in the input gradient dx = dy W + dt A. The [M, out] base output is never written and re-read."""

    @staticmethod
    def forward(ctx, x, w, bias, a, b, scale, residual, quant):
        x2 = _flat2d(x)
        r2 = _flat2d(residual) if residual is not None else None
        w_ref = w
        if quant is not None:
            w = quant.dequantize(shared=True)                # consumed by the GEMM below, not kept
        t = K.gemm(x2, a, alpha=scale)                       # [M, r]
        y = torch.empty((*x.shape[:-1], w.shape[0]), dtype=torch.bfloat16, device=x.device)
        K.gemm_ext(x2, w, t, b, out=y.view(-1, w.shape[0]), bias=bias, residual=r2)
        ctx.save_for_backward(x2, None if quant is not None else w, a, b, t)
        ctx.scale, ctx.x_shape, ctx.quant = scale, x.shape, quant
        ctx.refs = (w_ref, bias, a, b)
        ctx.has_res = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w, a, b, t = ctx.saved_tensors
        w_ref, bias_ref, a_ref, b_ref = ctx.refs
        dy2 = _flat2d(dy)
        if ctx.quant is not None and ctx.needs_input_grad[0]:
            w = ctx.quant.dequantize(shared=True)            # expanded again for the input gradient
        dt = K.gemm(dy2, b, b_mn=True, alpha=ctx.scale)      # [M, r] = scale * dy B
        db = K.gemm(dy2, t, a_mn=True, b_mn=True)            # [out, r] (t carries the scale)
        da = K.gemm(dt, x2, a_mn=True, b_mn=True)            # [r, in]
        dx = dw = dbias = None
        if ctx.needs_input_grad[0]:
            dx = K.gemm_ext(dy2, w, dt, a, b_mn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            mg = getattr(w_ref, "main_grad", None)
            if mg is not None:
                K.gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, accumulate=True)
                w_ref.grad_added_to_main_grad = True
            else:
                dw = K.gemm(dy2, x2, a_mn=True, b_mn=True)
        if bias_ref is not None and ctx.needs_input_grad[2]:
            dbias = _deliver_grad(bias_ref, dy2.float().sum(0).to(dy.dtype))
        return dx, dw, dbias, _deliver_grad(a_ref, da), _deliver_grad(b_ref, db), None, dy if ctx.has_res else None, None


def lora_linear(x, w, bias, a, b, scale: float, residual=None, quant=None):
    """x W^T + scale * x A^T B^T (+ bias) (+ residual); w [out, in], a [r, in], b [out, r]. `quant`: the base weight as
    a 4-bit object with `dequantize(shared=...)` instead of `w` (QLoRA): it is expanded for the forward GEMM and again
    for the input-gradient GEMM, never stored in expanded form."""
    r = a.shape[0]
    w_dtype = w.dtype if w is not None else quant.dtype
    if _native(x) and w_dtype == torch.bfloat16 and a.dtype == torch.bfloat16 and r % 8 == 0 and x.shape[-1] % 8 == 0:
        return _LoraLinearFn.apply(x, w, bias, a, b, float(scale), residual, quant)
    if w is None:
        w = quant.dequantize()
    y = lora_delta(x, a, b, linear(x, w, bias), scale)
    return y if residual is None else y + residual


def lora_delta(x, a, b, base, scale: float):
    """base + scale * x A^T B^T (LoRA update added to an already computed projection)."""
    r = a.shape[0]
    if _native(x) and a.dtype == torch.bfloat16 and r % 8 == 0 and x.shape[-1] % 8 == 0:
        return _LoraDeltaFn.apply(x, a, b, base, float(scale))
    t = torch.nn.functional.linear(x, a.to(x.dtype))
    return base + scale * torch.nn.functional.linear(t, b.to(x.dtype))


# ---------------------------------------------------------------------------- rmsnorm
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, add_one):
        x2 = _flat2d(x)
        y = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
        _, rstd = K.rmsnorm_fwd(x2, w, eps, add_one, out=y.view(x2.shape))
        ctx.save_for_backward(x2, w, rstd)
        ctx.add_one = add_one
        ctx.w_ref = w
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        want_dw = ctx.needs_input_grad[1]
        dx, dw = K.rmsnorm_bwd(_flat2d(dy), x2, w, rstd, ctx.add_one, want_dw=want_dw)
        if dw is not None:
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:
                mg.add_(dw.to(mg.dtype))
                ctx.w_ref.grad_added_to_main_grad = True
                dw = None
            else:
                dw = dw.to(w.dtype)
        return dx.view(dy.shape), dw, None, None


def rmsnorm(x, w, eps: float = 1e-6, add_one: bool = False):
    if _native(x) and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _RMSNormFn.apply(x, w, eps, add_one)
    return R.rmsnorm_ref(x, w, eps, add_one)


# ------------------------------------------------------------------------------- rope
class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, positions, cos, sin):
        # x [B,T,heads,H] contiguous; rotated in place (x is a fresh projection output)
        B, T, Hh, H = x.shape
        K.rope_(x.view(B * T, Hh, H), positions.reshape(-1), cos, sin)
        ctx.save_for_backward(positions, cos, sin)
        ctx.mark_dirty(x)
        return x

    @staticmethod
    def backward(ctx, dy):
        positions, cos, sin = ctx.saved_tensors
        dy = dy.contiguous()
        B, T, Hh, H = dy.shape
        K.rope_(dy.view(B * T, Hh, H), positions.reshape(-1), cos, sin, backward=True)
        return dy, None, None, None


def rope(x, positions, cos, sin):
    """Half-split rotary embedding on x [B,T,heads,H]; positions int [B,T]."""
    if _native(x) and x.is_contiguous() and x.shape[-1] % 4 == 0:
        pos = positions if positions.dtype == torch.int32 else positions.to(torch.int32)
        if x.requires_grad or not x.is_leaf:
            x = x.clone() if x.is_leaf else x
        return _RopeFn.apply(x, pos.contiguous(), cos, sin)
    return R.rope_ref(x, positions, cos, sin)


# -------------------------------------------------------------------------------- glu
class _GluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, u, kind):
        g2, u2 = _flat2d(g), _flat2d(u)
        h = K.glu_fwd(g2, u2, kind)
        ctx.save_for_backward(g2, u2)
        ctx.kind = kind
        return h.view(g.shape)

    @staticmethod
    def backward(ctx, dh):
        g2, u2 = ctx.saved_tensors
        dg, du = K.glu_bwd(_flat2d(dh), g2, u2, ctx.kind)
        return dg.view(dh.shape), du.view(dh.shape), None


def glu(g, u, kind: str = "silu"):
    """act(g) * u with act = SiLU (SwiGLU) or tanh-GELU (GeGLU)."""
    if _native(g) and g.shape[-1] % 8 == 0:
        return _GluFn.apply(g, u, K.GLU_SILU if kind == "silu" else K.GLU_GELU)
    return R.glu_ref(g, u, kind)


# -------------------------------------------------------------------------- attention
class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, causal, window, softcap, q_off, seg_q, seg_k):
        o, lse = K.attn_fwd(q, k, v, scale=scale, causal=causal, window=window, softcap=softcap, q_off=q_off,
                            seg_q=seg_q, seg_k=seg_k)
        ctx.save_for_backward(q, k, v, o, lse, seg_q, seg_k)
        ctx.cfg = (scale, causal, window, softcap, q_off)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, seg_q, seg_k = ctx.saved_tensors
        scale, causal, window, softcap, q_off = ctx.cfg
        do = do.contiguous()
        dq, dk, dv = K.attn_bwd(do, q, k, v, o, lse, scale=scale, causal=causal, window=window, softcap=softcap,
                                q_off=q_off, seg_q=seg_q, seg_k=seg_k)
        return dq, dk, dv, None, None, None, None, None, None, None


def attention(q, k, v, *, scale: float, causal: bool = True, window: int = 0, softcap: float = 0.0,
              q_off: int | None = None, seg_q=None, seg_k=None):
    """Flash attention. q [B,Tq,N,H]; k, v [B,Tk,KH,H]; segment ids int32 [B,T] (equal ids attend)."""
    H = q.shape[-1]
    if _native(q) and H in (64, 128, 256):
        q, k, v = (t if t.is_contiguous() else t.contiguous() for t in (q, k, v))
        if seg_q is not None:
            seg_q = seg_q.to(torch.int32).contiguous()
            seg_k = seg_k.to(torch.int32).contiguous()
        return _AttnFn.apply(q, k, v, float(scale), bool(causal), int(window or 0), float(softcap or 0.0), q_off,
                             seg_q, seg_k)
    if _library_mode and q.is_cuda and causal and not window and not softcap and seg_q is None and q_off is None \
            and q.shape[1] == k.shape[1]:
        o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                             is_causal=True, scale=scale, enable_gqa=True)
        return o.transpose(1, 2).contiguous()
    return R.attention_ref(q, k, v, scale=scale, causal=causal, window=window or 0, softcap=softcap or 0.0,
                           q_off=q_off, seg_q=seg_q, seg_k=seg_k)


# -------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, scale):
        ids32 = ids.reshape(-1).to(torch.int32).contiguous()
        out = K.embedding_fwd(ids32, table, scale)
        ctx.save_for_backward(ids32)
        ctx.table_ref = table
        ctx.scale = scale
        return out.view(*ids.shape, table.shape[1])

    @staticmethod
    def backward(ctx, dout):
        (ids32,) = ctx.saved_tensors
        table = ctx.table_ref
        d2 = _flat2d(dout)
        mg = getattr(table, "main_grad", None)
        if mg is not None and mg.dtype == torch.bfloat16:
            K.embedding_bwd(ids32, d2, mg, ctx.scale)
            table.grad_added_to_main_grad = True
            return None, None, None
        dt = torch.zeros_like(table)
        K.embedding_bwd(ids32, d2, dt, ctx.scale)
        if mg is not None:
            mg.add_(dt.to(mg.dtype))
            table.grad_added_to_main_grad = True
            return None, None, None
        return None, dt, None


def embedding(ids, table, scale: float = 1.0):
    if table.is_cuda and table.dtype == torch.bfloat16 and table.shape[1] % 8 == 0 and not _library_mode:
        return _EmbeddingFn.apply(ids, table, float(scale))
    out = torch.nn.functional.embedding(ids.long(), table)
    return out * scale if scale != 1.0 else out


# ---------------------------------------------------------------- lm_head log-probs
class _LmHeadLogprobFn(torch.autograd.Function):
    """lm_head -> log-softmax -> gather without logits in memory: the forward keeps per-row statistics only, the
    backward recomputes the logits chunk by chunk and holds a bf16 [chunk, V] gradient between its GEMMs. Problems too
    small for the two-SM GEMM use an fp32 [chunk, V] logits buffer instead."""

    @staticmethod
    def forward(ctx, h, w, targets, softcap, temperature, want_entropy, chunk):
        h2 = _flat2d(h)
        rows, V = h2.shape[0], w.shape[0]
        tg = targets.reshape(-1).to(torch.int32).contiguous()
        logp = torch.empty(rows, dtype=torch.float32, device=h.device)
        lse = torch.empty_like(logp)
        ent = torch.empty_like(logp) if want_entropy else None
        # fused path: the two-SM GEMM's epilogue reduces each 256-column tile to softmax statistics, no logits in memory
        fused = K.lm_head_lse(h2, w, tg, softcap=softcap, temperature=temperature, logp=logp, lse=lse, entropy=ent)
        buf = None if fused else torch.empty((min(chunk, max(rows, 1)), V), dtype=torch.float32, device=h.device)
        for s0 in range(0, rows if not fused else 0, chunk):
            n = min(chunk, rows - s0)
            z = buf[:n]
            K.gemm(h2[s0:s0 + n], w, out=z)
            lp, ls, en = K.logsoftmax_gather(z, tg[s0:s0 + n], softcap=softcap, temperature=temperature,
                                             want_entropy=want_entropy)
            logp[s0:s0 + n] = lp
            lse[s0:s0 + n] = ls
            if want_entropy:
                ent[s0:s0 + n] = en
        ctx.save_for_backward(h2, w, tg, lse, ent if want_entropy else None)
        ctx.cfg = (softcap, temperature, want_entropy, chunk)
        ctx.h_shape = h.shape
        ctx.w_ref = w
        out_shape = targets.shape
        if want_entropy:
            return logp.view(out_shape), ent.view(out_shape)
        return logp.view(out_shape), None

    @staticmethod
    def backward(ctx, dlogp, dent):
        h2, w, tg, lse, ent = ctx.saved_tensors
        softcap, temperature, want_entropy, chunk = ctx.cfg
        rows, V = h2.shape[0], w.shape[0]
        dlogp = dlogp.reshape(-1).float().contiguous() if dlogp is not None else None
        dent = dent.reshape(-1).float().contiguous() if (dent is not None and want_entropy) else None
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dh = torch.empty_like(h2) if need_dh else None
        mg = getattr(ctx.w_ref, "main_grad", None) if need_dw else None
        dw = None
        if need_dw and mg is None:
            dw = torch.zeros((V, h2.shape[1]), dtype=torch.float32, device=h2.device)
        zbuf = None
        dbuf = torch.empty((min(chunk, max(rows, 1)), V), dtype=torch.bfloat16, device=h2.device)
        for s0 in range(0, rows, chunk):
            n = min(chunk, rows - s0)
            sl = slice(s0, s0 + n)
            row_args = (tg[sl], lse[sl], ent[sl] if ent is not None else None, dlogp[sl] if dlogp is not None else None,
                        dent[sl] if dent is not None else None)
            dz = dbuf[:n]
            # the GEMM that recomputes the chunk's logits turns them into their gradient in its epilogue
            if not K.lm_head_dlogits(h2[sl], w, *row_args, softcap=softcap, temperature=temperature, out=dz):
                if zbuf is None:
                    zbuf = torch.empty((min(chunk, max(rows, 1)), V), dtype=torch.float32, device=h2.device)
                z = zbuf[:n]
                K.gemm(h2[sl], w, out=z)
                K.dlogits(z, *row_args, softcap=softcap, temperature=temperature, out=dz)
            if need_dh:
                K.gemm(dz, w, b_mn=True, out=dh[s0:s0 + n])
            if need_dw:
                K.gemm(dz, h2[s0:s0 + n], a_mn=True, b_mn=True, out=mg if mg is not None else dw, accumulate=True)
        if mg is not None:
            ctx.w_ref.grad_added_to_main_grad = True
        elif dw is not None:
            dw = dw.to(w.dtype)
        return (dh.view(ctx.h_shape) if dh is not None else None), dw, None, None, None, None, None


def lm_head_logprobs(h, w, targets, *, softcap: float = 0.0, temperature: float = 1.0, want_entropy: bool = False,
                     chunk: int = 2048):
    """log p(target | h) per token, optionally with the entropy of the predictive distribution.

    h [..., D], w [V, D], targets [...] (negative = ignore). Returns (logp fp32, entropy fp32 | None).
    """
    if _native(h) and w.dtype == torch.bfloat16 and h.shape[-1] % 8 == 0:
        return _LmHeadLogprobFn.apply(h, w, targets, float(softcap or 0.0), float(temperature), bool(want_entropy),
                                      int(chunk) if chunk and chunk > 0 else 2048)
    h2 = h.reshape(-1, h.shape[-1])
    if _library_mode and h.is_cuda and h.dtype == torch.bfloat16:
        # what a stock PyTorch trainer does: bf16 logits from the library GEMM, fp32 log-softmax, row chunks
        lps, ents = [], []
        tg_all = targets.reshape(-1).long()
        for s0 in range(0, h2.shape[0], chunk or h2.shape[0]):
            z = torch.nn.functional.linear(h2[s0:s0 + chunk], w).float()
            if softcap and softcap > 0:
                z = softcap * torch.tanh(z / softcap)
            lsm = torch.log_softmax(z / temperature, dim=-1)
            tg = tg_all[s0:s0 + chunk]
            lps.append(lsm.gather(1, tg.clamp(0, w.shape[0] - 1)[:, None])[:, 0] * (tg >= 0))
            if want_entropy:
                ents.append(-(lsm.exp() * lsm).sum(-1))
        ent = torch.cat(ents).view(targets.shape) if want_entropy else None
        return torch.cat(lps).view(targets.shape), ent
    logp, ent = R.lm_head_logprobs_ref(h2, w, targets.reshape(-1), softcap=softcap or 0.0, temperature=temperature,
                                       want_entropy=want_entropy, chunk=chunk)
    return logp.view(targets.shape), (ent.view(targets.shape) if ent is not None else None)


def lm_head_logits(h, w, *, softcap: float = 0.0):
    """Full fp32 logits (sampling / small models only)."""
    if _native(h) and w.dtype == torch.bfloat16 and h.shape[-1] % 8 == 0 and not (h.requires_grad or w.requires_grad):
        z = K.gemm(_flat2d(h), w, out_dtype=torch.float32).view(*h.shape[:-1], w.shape[0])
    else:
        z = torch.nn.functional.linear(h, w.to(h.dtype)).float()
    if softcap and softcap > 0:
        z = softcap * torch.tanh(z / softcap)
    return z
