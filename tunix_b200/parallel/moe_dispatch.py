"""Expert computation for MoE layers: token permutation, per-expert SwiGLU, weighted combine.

Single-rank path: tokens are sorted by expert once, each expert runs its gate/up/down
projections on a contiguous row slice (tcgen05 GEMMs on CUDA), and outputs are scattered
back with the routing weights. With an expert-parallel group attached to the layer
(`layer.ep_group`), `parallel/ep.py` performs the dispatch / combine exchange around the
same per-expert kernel.

Reference semantics: tunix/models/qwen3/model.py:894-1149 (dense fallback :911-939).
"""
from __future__ import annotations

import torch

from ..ops import functional as F


def _experts_on_rows(layer, xs: torch.Tensor, counts, first_expert: int = 0) -> torch.Tensor:
    """xs: rows sorted by (local) expert; counts[e] rows belong to expert first_expert+e."""
    out = torch.empty_like(xs)
    start = 0
    kind = layer.cfg.activation
    for e, n in enumerate(counts):
        n = int(n)
        if n == 0:
            continue
        rows = xs[start:start + n]
        g = F.linear(rows, layer.gate_proj[first_expert + e])
        u = F.linear(rows, layer.up_proj[first_expert + e])
        out[start:start + n] = F.linear(F.glu(g, u, kind), layer.down_proj[first_expert + e])
        start += n
    return out


def expert_forward(layer, x: torch.Tensor, weights: torch.Tensor, idx: torch.Tensor, recompute: bool = False) -> torch.Tensor:
    """x [T, D]; weights, idx [T, k]. Returns sum_k w * expert_{idx}(x)  [T, D]."""
    if getattr(layer, "ep", None) is not None and layer.ep.world > 1:
        from . import ep
        return ep.expert_parallel_forward(layer, x, weights, idx, recompute=recompute)
    T, D = x.shape
    k = idx.shape[1]
    E = layer.cfg.num_experts
    if x.is_cuda and x.dtype == torch.bfloat16 and D % 64 == 0 and layer.cfg.moe_hidden_dim % 64 == 0 and E <= 1024:
        from ..ops import moe as moe_ops
        return moe_ops.experts(x, weights, idx, layer.gate_proj, layer.up_proj, layer.down_proj, None,
                               layer.cfg.activation)
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    token_of = torch.div(order, k, rounding_mode="floor")
    xs = x.index_select(0, token_of)
    counts = torch.bincount(flat, minlength=E).tolist()
    ys = _experts_on_rows(layer, xs, counts)
    ys = ys * weights.reshape(-1)[order].unsqueeze(-1).to(ys.dtype)
    out = torch.zeros_like(x)
    out.index_add_(0, token_of, ys)
    return out
