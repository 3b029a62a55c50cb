"""Context parallelism: the sequence axis of the activations sharded over a group ("sp" mesh axis).

The reference shards activations along the sequence with the `sp` axis of its mesh and lets the compiler gather
keys and values where attention needs them (tunix/models/llama3/model.py:47-82 sharding rules; mesh axes in
tunix/cli/base_config.yaml). Here the same split is explicit:

* every rank of the group receives the same batch and keeps tokens [r*T/w, (r+1)*T/w) of every sequence: the
  embedding, every projection, norm, MLP and the lm_head run on T/w tokens per sequence;
* attention gathers K and V (after RoPE) along the sequence over the group and attends its own queries to the keys
  at or before them: `q_off = r*T/w` in the flash kernel, keys past the rank's last token are not even read. The
  backward of the gather is a reduce-scatter, so dK / dV contributions of later ranks come back to the owner;
* parameters are replicated over the group, so their gradients are summed over it exactly as over a data-parallel
  group (the sharded optimizer over the whole world does that);
* the next-token targets are shifted BEFORE the split (`shift_and_slice`), so the last token of a slice is scored
  against the first token of the next slice.

Causal attention over contiguous slices loads the ranks unevenly (rank r reads (r+1)/w of the keys); a zigzag
split would even that out and is not built. The gather is a library collective (NCCL / gloo); it moves
2 * B * T * kv_heads * head_dim elements per layer, small next to the projections it saves.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class _GatherSeq(torch.autograd.Function):
    """[B, T/w, ...] -> [B, T, ...] over the group; backward: sum over ranks of the slice that belongs to this rank."""

    @staticmethod
    def forward(ctx, x, group, world, rank):
        ctx.group, ctx.world, ctx.rank = group, world, rank
        x = x.contiguous()
        out = torch.empty((world * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device)     # rank-major
        dist.all_gather_into_tensor(out, x, group=group)
        return out.view(world, *x.shape).transpose(0, 1).reshape(x.shape[0], world * x.shape[1], *x.shape[2:])

    @staticmethod
    def backward(ctx, g):
        B, T = g.shape[:2]
        w = ctx.world
        parts = g.reshape(B, w, T // w, *g.shape[2:]).transpose(0, 1).contiguous()      # [w, B, T/w, ...]
        out = torch.empty_like(parts[0])
        if dist.get_backend(ctx.group) == "gloo":           # gloo has no reduce-scatter: reduce, then keep the own slice
            dist.all_reduce(parts, group=ctx.group)
            out.copy_(parts[ctx.rank])
        else:
            dist.reduce_scatter_tensor(out, parts.view(w * B, *parts.shape[2:]), op=dist.ReduceOp.SUM, group=ctx.group)
        return out, None, None, None


class ContextParallel:
    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    # ------------------------------------------------------------------ slicing
    def local_len(self, T: int) -> int:
        if T % self.world:
            raise ValueError(f"sequence length {T} is not divisible by the context-parallel size {self.world}")
        return T // self.world

    def slice_seq(self, t: Optional[torch.Tensor], dim: int = 1) -> Optional[torch.Tensor]:
        """This rank's tokens of a [B, T, ...] tensor."""
        if t is None or self.world == 1:
            return t
        n = self.local_len(t.shape[dim])
        return t.narrow(dim, self.rank * n, n)

    def shift_and_slice(self, tokens: torch.Tensor, mask: torch.Tensor):
        """(targets, mask) for this rank's positions: position t is scored against token t+1 of the FULL sequence,
        the last position of the sequence against nothing."""
        targets = torch.cat([tokens[:, 1:], tokens.new_zeros(tokens.shape[0], 1)], 1)
        m = torch.cat([mask[:, 1:], mask.new_zeros(mask.shape[0], 1)], 1)
        return self.slice_seq(targets), self.slice_seq(m)

    # --------------------------------------------------------------- attention
    def gather_seq(self, x: torch.Tensor) -> torch.Tensor:
        """All ranks' slices of [B, T/w, ...] joined along the sequence (differentiable)."""
        if self.world == 1:
            return x
        if torch.is_grad_enabled() and x.requires_grad:
            return _GatherSeq.apply(x, self.group, self.world, self.rank)
        return _GatherSeq.forward(_NoCtx(), x, self.group, self.world, self.rank)

    def keys_for_local_queries(self, k, v, segment_ids):
        """(k, v, seg_k, q_off): keys / values of the whole sequence up to this rank's last token, the matching
        segment ids, and the position of this rank's first query among them."""
        Tl = k.shape[1]
        end = (self.rank + 1) * Tl
        k_all, v_all = self.gather_seq(k)[:, :end], self.gather_seq(v)[:, :end]
        seg_k = None
        if segment_ids is not None:
            seg_k = self.gather_seq(segment_ids.detach())[:, :end].contiguous()
        return k_all, v_all, seg_k, self.rank * Tl


class _NoCtx:
    pass


def apply_context_parallel(model, group=None) -> ContextParallel:
    """Shard the sequence axis of `model`'s activations over `group`. The model then expects the same full batch on
    every rank of the group and returns hidden states for this rank's tokens."""
    from ..models.transformer import Attention, Transformer
    if not isinstance(model, Transformer):
        raise NotImplementedError("context parallelism covers the generic decoder")
    if getattr(model, "tp", None) is not None:
        raise NotImplementedError("context parallelism with tensor parallelism on the same model is not built")
    ctx = ContextParallel(group)
    model.cp = ctx
    for m in model.modules():
        if isinstance(m, Attention):
            m.cp = ctx
    return ctx
