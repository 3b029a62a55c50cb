"""Expert computation of a mixture-of-experts layer on the grouped tcgen05 GEMM.

Routing (softmax / top-k / renormalise) stays in PyTorch on the small `[tokens, experts]` tensors so that
autograd differentiates it; everything that touches `[tokens * k, D]` data runs in the kernels of
`csrc/moe.cu` and the grouped mode of `csrc/gemm.cu`. No step reads a count back to the host.

Layout: the `k` copies of each token are permuted into per-expert row segments that start on multiples of
128 rows and are zero padded (`route_positions`). Forward: scatter -> gate / up grouped GEMM -> gated
activation -> down grouped GEMM -> weighted gather-sum. Backward mirrors it, with the weight gradients as
grouped GEMMs contracted over each expert's segment, accumulated straight into `main_grad` when present.

Reference semantics: tunix/models/qwen3/model.py:941-1149 (sort, ragged_dot x3, unsort, weighted sum).
"""
from __future__ import annotations

import torch

from . import kernels as K


def route_positions(idx: torch.Tensor, num_experts: int):
    """idx [T, k] expert ids -> (counts int32 [E], seg_off int32 [E+1], pos int32 [T, k], max_rows).

    pos[t, j] is the row of the permuted buffer that holds copy j of token t; rows of one expert are ordered
    by (token, slot), so the layout is deterministic. max_rows bounds seg_off[E] without reading it."""
    T, k = idx.shape
    flat = idx.reshape(-1).long()
    # scatter-add instead of bincount: no read-back of the largest id, so the step stays capturable in a CUDA graph
    counts = torch.zeros(num_experts, dtype=torch.int64, device=idx.device).scatter_add_(0, flat, torch.ones_like(flat))
    padded = (counts + 127) // 128 * 128
    seg_off = torch.zeros(num_experts + 1, dtype=torch.int64, device=idx.device)
    seg_off[1:] = torch.cumsum(padded, 0)
    order = torch.argsort(flat, stable=True)
    sorted_e = flat[order]
    starts = torch.cumsum(counts, 0) - counts
    rank = torch.arange(flat.numel(), device=idx.device) - starts[sorted_e]
    pos = torch.empty_like(flat)
    pos[order] = seg_off[sorted_e] + rank
    max_rows = ((T * k + num_experts * 127 + 127) // 128) * 128
    return counts.int(), seg_off.int(), pos.int().view(T, k), max_rows


class _ExpertsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, wts, pos, seg_off, counts, max_rows, gate_w, up_w, down_w, residual, kind):
        T, D = x.shape
        E, Fd, _ = gate_w.shape
        dev = x.device
        xp = torch.empty((max_rows, D), dtype=torch.bfloat16, device=dev)
        K.moe_zero_pad(xp, seg_off, counts)
        K.moe_scatter_rows(x, pos, None, xp)
        t_up = K.moe_tiles_rows(seg_off, max_rows, Fd, D, Fd)          # [R, F] <- xp [R, D] x W[e] [F, D]
        t_down = K.moe_tiles_rows(seg_off, max_rows, D, Fd, D)         # [R, D] <- h  [R, F] x W[e] [D, F]
        g = torch.empty((max_rows, Fd), dtype=torch.bfloat16, device=dev)
        u = torch.empty_like(g)
        K.gemm_grouped(xp, gate_w.view(E * Fd, D), g, Fd, t_up)
        K.gemm_grouped(xp, up_w.view(E * Fd, D), u, Fd, t_up)
        h = K.glu_fwd(g, u, kind)
        y = torch.empty((max_rows, D), dtype=torch.bfloat16, device=dev)
        K.gemm_grouped(h, down_w.view(E * D, Fd), y, D, t_down)
        out = K.moe_gather_sum(y, pos, wts, residual)
        ctx.save_for_backward(xp, g, u, y, wts, pos, seg_off, counts, gate_w, up_w, down_w)
        ctx.kind, ctx.max_rows, ctx.has_res = kind, max_rows, residual is not None
        ctx.w_refs = (gate_w, up_w, down_w)
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable      # the saved buffers are overwritten below: one backward per forward
    def backward(ctx, dout):
        xp, g, u, y, wts, pos, seg_off, counts, gate_w, up_w, down_w = ctx.saved_tensors
        E, Fd, D = gate_w.shape
        R, dev = ctx.max_rows, dout.device
        dout = dout.contiguous()
        dwts = K.moe_dot_rows(dout, y, pos)
        dy = y                                             # y is dead after the dot: reuse its storage
        K.moe_zero_pad(dy, seg_off, counts)
        K.moe_scatter_rows(dout, pos, wts, dy)
        h = K.glu_fwd(g, u, ctx.kind)

        def wgrad(a, b, w_ref, m_out, n_out):
            tl = K.moe_tiles_expert(seg_off, m_out, n_out)
            mg = getattr(w_ref, "main_grad", None)
            if mg is not None:
                K.gemm_grouped(a, b, mg.view(E, m_out, n_out), n_out, tl, a_mn=True, b_mn=True, accumulate=True)
                w_ref.grad_added_to_main_grad = True
                return None
            dw = torch.empty((E, m_out, n_out), dtype=torch.bfloat16, device=dev)
            K.gemm_grouped(a, b, dw, n_out, tl, a_mn=True, b_mn=True)
            return dw

        gw_ref, uw_ref, dw_ref = ctx.w_refs
        d_down = wgrad(dy, h, dw_ref, D, Fd) if ctx.needs_input_grad[8] else None
        # dh [R, F] = dy [R, D] x W_down[e] ([D, F], contracted over D: MN-major B)
        t_dh = K.moe_tiles_rows(seg_off, R, Fd, D, D)
        dh = h
        K.gemm_grouped(dy, down_w.view(E * D, Fd), dh, Fd, t_dh, b_mn=True)
        dg, du = K.glu_bwd(dh, g, u, ctx.kind, inplace=True)
        d_gate = wgrad(dg, xp, gw_ref, Fd, D) if ctx.needs_input_grad[6] else None
        d_up = wgrad(du, xp, uw_ref, Fd, D) if ctx.needs_input_grad[7] else None
        dx = None
        if ctx.needs_input_grad[0]:
            # dxp [R, D] = dg x W_gate[e] + du x W_up[e] ([F, D], contracted over F)
            t_dx = K.moe_tiles_rows(seg_off, R, D, Fd, Fd)
            dxp = xp
            K.gemm_grouped(dg, gate_w.view(E * Fd, D), dxp, D, t_dx, b_mn=True)
            K.gemm_grouped(du, up_w.view(E * Fd, D), dxp, D, t_dx, b_mn=True, accumulate=True)
            dx = K.moe_gather_sum(dxp, pos, None)
        dres = dout if ctx.has_res else None
        return dx, dwts, None, None, None, None, d_gate, d_up, d_down, dres, None


def experts(x, wts, idx, gate_w, up_w, down_w, residual=None, kind: str = "silu"):
    """sum_j wts[t, j] * expert_{idx[t, j]}(x[t]) (+ residual). x [T, D] bf16; wts [T, k] (any float dtype,
    differentiable); idx [T, k]; expert weights stacked [E, F, D], [E, F, D], [E, D, F]."""
    E, Fd, D = gate_w.shape
    assert D % 64 == 0 and Fd % 64 == 0, "grouped GEMM contracts in 64-element blocks"
    counts, seg_off, pos, max_rows = route_positions(idx, E)
    return _ExpertsFn.apply(x.contiguous(), wts.float().contiguous(), pos, seg_off, counts, max_rows, gate_w, up_w,
                            down_w, residual, K.GLU_SILU if kind == "silu" else K.GLU_GELU)


class _LocalExpertsFn(torch.autograd.Function):
    """Experts of one rank on rows that are already in expert order (expert parallelism): the routing weight
    arrives per row and is applied to the activation before the down projection, so the rows that travel back
    are ready to be summed, and its gradient <dy, y> is formed here as <dy W_down, h> without keeping y."""

    @staticmethod
    def forward(ctx, xp, wrow, seg_off, counts, gate_w, up_w, down_w, kind, recompute=False):
        R, D = xp.shape
        E, Fd, _ = gate_w.shape
        dev = xp.device
        t_up = K.moe_tiles_rows(seg_off, R, Fd, D, Fd)
        t_down = K.moe_tiles_rows(seg_off, R, D, Fd, D)
        g = torch.empty((R, Fd), dtype=torch.bfloat16, device=dev)
        u = torch.empty_like(g)
        K.gemm_grouped(xp, gate_w.view(E * Fd, D), g, Fd, t_up)
        K.gemm_grouped(xp, up_w.view(E * Fd, D), u, Fd, t_up)
        hs = K.moe_row_scale(K.glu_fwd(g, u, kind), wrow)
        y = torch.empty((R, D), dtype=torch.bfloat16, device=dev)
        K.gemm_grouped(hs, down_w.view(E * D, Fd), y, D, t_down)
        # `recompute`: keep only the dispatched rows; gate / up are rebuilt in backward by two local grouped GEMMs.
        # This is activation recomputation that stays on this rank: the rows are not exchanged a second time.
        if recompute:
            ctx.save_for_backward(xp, wrow, seg_off, gate_w, up_w, down_w)
        else:
            ctx.save_for_backward(xp, g, u, wrow, seg_off, gate_w, up_w, down_w)
        ctx.kind, ctx.recompute = kind, recompute
        ctx.w_refs = (gate_w, up_w, down_w)
        return y

    @staticmethod
    @torch.autograd.function.once_differentiable      # the saved buffers are overwritten below: one backward per forward
    def backward(ctx, dy):
        if ctx.recompute:
            xp, wrow, seg_off, gate_w, up_w, down_w = ctx.saved_tensors
            E, Fd, D = gate_w.shape
            t_up = K.moe_tiles_rows(seg_off, xp.shape[0], Fd, D, Fd)
            g = torch.empty((xp.shape[0], Fd), dtype=torch.bfloat16, device=xp.device)
            u = torch.empty_like(g)
            K.gemm_grouped(xp, gate_w.view(E * Fd, D), g, Fd, t_up)
            K.gemm_grouped(xp, up_w.view(E * Fd, D), u, Fd, t_up)
        else:
            xp, g, u, wrow, seg_off, gate_w, up_w, down_w = ctx.saved_tensors
        E, Fd, D = gate_w.shape
        R, dev = xp.shape[0], dy.device
        dy = dy.contiguous()
        h = K.glu_fwd(g, u, ctx.kind)

        def wgrad(a, b, w_ref, m_out, n_out):
            tl = K.moe_tiles_expert(seg_off, m_out, n_out)
            mg = getattr(w_ref, "main_grad", None)
            if mg is not None:
                K.gemm_grouped(a, b, mg.view(E, m_out, n_out), n_out, tl, a_mn=True, b_mn=True, accumulate=True)
                w_ref.grad_added_to_main_grad = True
                return None
            dw = torch.empty((E, m_out, n_out), dtype=torch.bfloat16, device=dev)
            K.gemm_grouped(a, b, dw, n_out, tl, a_mn=True, b_mn=True)
            return dw

        gw_ref, uw_ref, dw_ref = ctx.w_refs
        dhp = torch.empty((R, Fd), dtype=torch.bfloat16, device=dev)
        K.gemm_grouped(dy, down_w.view(E * D, Fd), dhp, Fd, K.moe_tiles_rows(seg_off, R, Fd, D, D), b_mn=True)
        dwrow = K.moe_row_dot(dhp, h) if ctx.needs_input_grad[1] else None
        d_down = None
        if ctx.needs_input_grad[6]:
            hs = K.moe_row_scale(h, wrow)
            d_down = wgrad(dy, hs, dw_ref, D, Fd)
        dh = K.moe_row_scale(dhp, wrow, out=dhp)
        dg, du = K.glu_bwd(dh, g, u, ctx.kind, inplace=True)
        d_gate = wgrad(dg, xp, gw_ref, Fd, D) if ctx.needs_input_grad[4] else None
        d_up = wgrad(du, xp, uw_ref, Fd, D) if ctx.needs_input_grad[5] else None
        dxp = None
        if ctx.needs_input_grad[0]:
            t_dx = K.moe_tiles_rows(seg_off, R, D, Fd, Fd)
            dxp = xp
            K.gemm_grouped(dg, gate_w.view(E * Fd, D), dxp, D, t_dx, b_mn=True)
            K.gemm_grouped(du, up_w.view(E * Fd, D), dxp, D, t_dx, b_mn=True, accumulate=True)
        return dxp, dwrow, None, None, d_gate, d_up, d_down, None, None


def local_experts(xp, wrow, seg_off, counts, gate_w, up_w, down_w, kind: str = "silu", recompute: bool = False):
    """y[r] = wrow[r] * expert_of_segment(r)(xp[r]) for rows laid out in this rank's expert segments."""
    return _LocalExpertsFn.apply(xp, wrow.float().contiguous(), seg_off, counts, gate_w, up_w, down_w,
                                 K.GLU_SILU if kind == "silu" else K.GLU_GELU, recompute)
