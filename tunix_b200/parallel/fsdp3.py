"""Weight-sharded data parallelism (ZeRO-3 style) on GEMMs that gather their own weights.

Every Linear weight is stored as this rank's block of rows only. The projection kernels pull the other
blocks from the peers while they compute (`csrc/gemm.cu`, all-gather fused into the tcgen05 GEMM; tiles of
the local block run first, tiles of a peer's block wait for that block's flags):

    forward    y  = x  @ gather(W_s)^T            gathered operand = B rows          (mode 2)
    backward   dx = dy @ gather(W_s)              gathered operand = the contraction (mode 3)
               dW_s = scatter_sum(dy^T @ x)       GEMM -> reduce-scatter over the ranks' token shards

so a full weight never exists outside the two per-shape staging buffers, the optimizer is the plain local
one on the shards (no parameter all-gather after the step), and parameters that stay whole (norms,
embeddings, biases) have their gradients summed with one all-reduce (`sync_replicated_grads`).

This is the counterpart of the reference's `fsdp` mesh axis on weights (`ffw_weight_df = (fsdp, tp)` etc.,
tunix/models/llama3/model.py:65-82), where XLA all-gathers each weight before its dot.
`parallel/fsdp.py` is the ZeRO-2 alternative (whole bf16 weights, sharded optimizer state).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from .tp import TPContext as CommContext, _wgrad_into  # noqa: F401  (same workspaces and primitives)


class _ShardedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, w_s, bias, residual2, comm: CommContext):
        y = comm.gemm_gather_w(x2, w_s, bias, residual2)
        ctx.save_for_backward(x2, w_s)
        ctx.comm, ctx.w_ref, ctx.has_bias, ctx.has_res = comm, w_s, bias is not None, residual2 is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w_s = ctx.saved_tensors
        comm = ctx.comm
        dy = dy.contiguous()
        dx = comm.gemm_gather_w_t(dy, w_s) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            g = comm.wgrad_scatter(dy, x2)
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:
                mg.add_(g.to(mg.dtype))
                ctx.w_ref.grad_added_to_main_grad = True
            else:
                dw = g
        db = dy.float().sum(0).to(dy.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db, (dy if ctx.has_res else None), None


def sharded_linear(x, w_s, bias, residual, comm: CommContext):
    lead = x.shape[:-1]
    r2 = residual.reshape(-1, residual.shape[-1]) if residual is not None else None
    y = _ShardedLinearFn.apply(x.reshape(-1, x.shape[-1]), w_s, bias, r2, comm)
    return y.view(*lead, y.shape[-1])


def apply_weight_sharding(model, comm: CommContext, min_rows: int = 1):
    """Replace every Linear weight of a Transformer by this rank's block of rows (out_features must divide by
    the group size; others stay whole). Returns the model; `model.dp_shard` carries the context."""
    W, r = comm.world, comm.rank
    from ..models.transformer import Linear
    with torch.no_grad():
        for mod in model.modules():
            if isinstance(mod, Linear) and mod.quant is None and mod.weight.shape[0] % W == 0 and \
                    mod.weight.shape[0] // W >= min_rows and getattr(mod, "tp", None) is None:
                n = mod.weight.shape[0] // W
                mod.weight = nn.Parameter(mod.weight.data[r * n:(r + 1) * n].clone(), requires_grad=mod.weight.requires_grad)
                mod.weight.dp_sharded = True
                mod.weight.shard_spec = (0, r, W)
                mod.weight.shard_group = comm.group
                mod.dp_shard = comm
    model.dp_shard = comm
    return model


def sync_replicated_grads(model, comm: CommContext) -> None:
    """Sum over the group the gradients of parameters that every rank holds whole."""
    if comm.world == 1:
        return
    grads = []
    for p in model.parameters():
        if getattr(p, "dp_sharded", False):
            continue
        g = getattr(p, "main_grad", None)
        g = g if g is not None else p.grad
        if g is not None:
            grads.append(g)
    for g in _coalesce_adjacent(grads):
        dist.all_reduce(g, group=comm.group)


def _coalesce_adjacent(tensors: list) -> list:
    """Contiguous tensors that follow each other in one storage (slots of an optimizer's flat gradient buffer) merged
    into one flat view per run, so that a model's whole parameters cost one collective per run instead of one per
    parameter (a mixture-of-experts layer: norms, attention projections and router form one run between the expert
    weights of neighbouring layers)."""
    items = [t for t in tensors if t.is_contiguous() and t.numel() > 0]
    rest = [t for t in tensors if not t.is_contiguous()]
    items.sort(key=lambda t: (t.untyped_storage().data_ptr(), t.storage_offset()))
    out, run = [], None            # run = [storage ptr, dtype, start offset, end offset, first tensor]
    for t in items:
        key, a, b = t.untyped_storage().data_ptr(), t.storage_offset(), t.storage_offset() + t.numel()
        if run is not None and run[0] == key and run[1] == t.dtype and run[3] == a:
            run[3] = b
            continue
        if run is not None:
            out.append(run)
        run = [key, t.dtype, a, b, t]
    if run is not None:
        out.append(run)
    views = [r[4].new_empty(0).set_(r[4].untyped_storage(), r[2], (r[3] - r[2],)) for r in out]
    return views + rest


def grad_sumsq(model, comm: CommContext) -> torch.Tensor:
    dev = next(model.parameters()).device
    sharded = torch.zeros((), dtype=torch.float32, device=dev)
    whole = torch.zeros((), dtype=torch.float32, device=dev)
    for p in model.parameters():
        g = getattr(p, "main_grad", None)
        g = g if g is not None else p.grad
        if g is None:
            continue
        s = g.float().pow(2).sum()
        if getattr(p, "dp_sharded", False):
            sharded += s
        else:
            whole += s
    if comm.world > 1:
        dist.all_reduce(sharded, group=comm.group)
    return (sharded + whole).reshape(1)
