"""Expert parallelism: each rank of the group keeps E / ep experts; tokens travel to their experts and back
over NVLink peer memory.

Every rank all-gathers the (tiny) routing tables, so all ranks derive the same global plan on the device: for
every (source rank, token, slot) the owner rank of its expert and the row it occupies in the owner's
expert-ordered buffer (segments start on multiples of 128 rows, zero padded, as `ops/moe.py` wants them).
The rows themselves move with two kernels of `csrc/moe.cu`, both plain P2P loads from symmetric memory:

    dispatch   owner pulls   xp[row]  = x_src[token]                       (moe_pull_rows)
    combine    source pulls  out[t]   = sum_j y_owner(j)[row(t, j)]        (moe_gather_sum_peer)

and their backward passes are each other: the owner pulls `dout` rows (combine backward), the source
gather-sums `dxp` rows (dispatch backward). The routing weight rides along as one fp32 per row and is applied
on the owner (`ops.moe.local_experts`), so rows that travel back are final and the weight's gradient is formed
where the expert output lives. One flag barrier (`symm.SymmBarrier`) stands between the writes and the pulls of an
exchange; the buffers alternate (`EPContext.workspace`), which makes a second barrier after the pulls unnecessary.

Without symmetric memory (CPU / gloo) the same result comes from all-gathering the tokens, computing the local
experts' share for all of them and reduce-scattering the sum: the path the CPU test runs.

Replaces the `shard_map` / ragged all-to-all expert-parallel branch of the reference's MoE block
(tunix/models/qwen3/model.py:1010-1149).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from . import symm


class EPContext:
    """`capacity_factor` (optional): receive buffers hold `capacity_factor x tokens x k` rows (plus one 128-row
    pad per local expert) instead of the exact count, so the routing plan needs no read-back from the device: no
    host synchronisation inside the layer. Slots that would land past the capacity are dropped (they contribute
    nothing, as in capacity-based MoE training) and `overflow` records that it happened; `raise_if_overflow()`
    reads it (one synchronisation, e.g. once per step)."""

    def __init__(self, group=None, device=None, capacity_factor=None):
        self.group = group
        self.capacity_factor = capacity_factor
        self.overflow = None
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self.fused = self.world > 1 and self.device.type == "cuda" and symm.symm_available(group)
        self.barrier = symm.SymmBarrier(self.device, group) if self.fused else None
        self._ws: dict = {}

    def raise_if_overflow(self) -> None:
        if self.overflow is not None and bool(self.overflow.item()):
            self.overflow = None
            raise RuntimeError("expert-parallel capacity exceeded: tokens were dropped; raise capacity_factor")

    def workspace(self, kind: str, rows: int, D: int) -> symm.SymmBuffer:
        """The symmetric buffer an exchange writes its rows into. Two buffers per (kind, shape) are handed out in
        turn, which is what lets an exchange run on ONE flag barrier (between "everyone has written" and the pulls):
        a buffer is written again two exchanges of its kind later, and a rank gets past the barrier in between only
        after every peer has arrived there, that is after every peer has finished pulling from the buffer. Every
        rank runs the same sequence of exchanges, so all ranks pick the same buffer."""
        key = (kind, rows, D)
        pair = self._ws.get(key)
        if pair is None:
            pair = self._ws[key] = [[symm.symm_empty(rows * D, torch.bfloat16, self.device, self.group, zero=True)
                                     for _ in range(2)], 0]
        pair[1] ^= 1
        return pair[0][pair[1]]


# ------------------------------------------------------------------------------- differentiable collectives
class _AllGather(torch.autograd.Function):
    """[n, ...] -> [W * n, ...]; backward sums the slices that belong to this rank."""

    @staticmethod
    def forward(ctx, x, group, world, rank):
        ctx.group, ctx.world, ctx.rank, ctx.n = group, world, rank, x.shape[0]
        out = torch.empty((world * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        if "nccl" in str(dist.get_backend(ctx.group)):
            out = torch.empty((ctx.n, *g.shape[1:]), dtype=g.dtype, device=g.device)
            dist.reduce_scatter_tensor(out, g, group=ctx.group)
            return out, None, None, None
        dist.all_reduce(g, group=ctx.group)
        return g[ctx.rank * ctx.n:(ctx.rank + 1) * ctx.n], None, None, None


class _ReduceScatter(torch.autograd.Function):
    """[W * n, ...] -> sum over ranks of this rank's [n, ...] slice; backward all-gathers."""

    @staticmethod
    def forward(ctx, x, group, world, rank):
        ctx.group, ctx.world = group, world
        n = x.shape[0] // world
        x = x.contiguous()
        if "nccl" in str(dist.get_backend(group)):
            out = torch.empty((n, *x.shape[1:]), dtype=x.dtype, device=x.device)
            dist.reduce_scatter_tensor(out, x, group=group)
            return out
        x = x.clone()
        dist.all_reduce(x, group=group)
        return x[rank * n:(rank + 1) * n].clone()

    @staticmethod
    def backward(ctx, g):
        out = torch.empty((ctx.world * g.shape[0], *g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None, None, None


# --------------------------------------------------------------------------------------------- the plan
class _Plan:
    """Global routing layout, identical on all ranks (built from the all-gathered expert ids)."""

    def __init__(self, idx_all: torch.Tensor, num_experts: int, ep: EPContext):
        W, r = ep.world, ep.rank
        WT, k = idx_all.shape
        T = WT // W
        E_loc = num_experts // W
        flat = idx_all.reshape(-1).long()
        # scatter-add, not bincount: bincount reads the largest id back to the host, a synchronisation per layer
        counts = torch.zeros(num_experts, dtype=torch.int64, device=flat.device).scatter_add_(0, flat, torch.ones_like(flat))
        padded = (counts + 127) // 128 * 128
        pad2 = padded.view(W, E_loc)
        seg_start = (torch.cumsum(pad2, 1) - pad2).reshape(-1)            # row where an expert starts on its owner
        order = torch.argsort(flat, stable=True)
        sorted_e = flat[order]
        starts = torch.cumsum(counts, 0) - counts
        rank_in = torch.arange(flat.numel(), device=flat.device) - starts[sorted_e]
        pos = torch.empty_like(flat)
        pos[order] = seg_start[sorted_e] + rank_in
        owner = flat // E_loc
        # worst case (every slot of every rank routed here): the size of the symmetric row workspace, which must be
        # the same on all ranks. What this rank actually receives is read back (the plan's one host synchronisation)
        # so that buffers and element-wise kernels cover those rows only: with 8 ranks the worst case is 8 times
        # the expected row count.
        self.max_rows = ((W * T * k + E_loc * 127 + 127) // 128) * 128
        if getattr(ep, "capacity_factor", None):
            # fixed capacity: nothing is read back. Segments are cut at the capacity, slots past it are dropped.
            self.rows = min(self.max_rows, ((int(ep.capacity_factor * T * k) + E_loc * 128 + 127) // 128) * 128)
            over = (pad2.sum(1) > self.rows).any()
            ep.overflow = over if ep.overflow is None else (ep.overflow | over)
            kept = pos < self.rows
            owner = torch.where(kept, owner, torch.full_like(owner, -1))      # dropped slots belong to nobody
        else:
            self.rows = max(128, int(pad2[r].sum().item()))
        # this rank as a source: where its slots live
        mine = slice(r * T * k, (r + 1) * T * k)
        self.dst_rank = owner[mine].int().view(T, k).contiguous()
        self.dst_pos = pos[mine].int().view(T, k).contiguous()
        # this rank as an owner: which (source, token) fills each of its rows. Slots owned elsewhere are sent to a
        # spare last entry instead of being compacted away (no `nonzero`, so no second host synchronisation).
        slots = torch.arange(flat.numel(), device=flat.device)
        self.own_dest = torch.where(owner == r, pos, torch.full_like(pos, self.rows))      # [W*T*k] row or `rows`
        self.src_rank = torch.full((self.rows + 1,), -1, dtype=torch.int32, device=flat.device).scatter_(
            0, self.own_dest, torch.div(slots, T * k, rounding_mode="floor").int())[:self.rows]
        self.src_rank = self.src_rank.contiguous()
        self.src_row = torch.zeros((self.rows + 1,), dtype=torch.int32, device=flat.device).scatter_(
            0, self.own_dest, (torch.div(slots, k, rounding_mode="floor") % T).int())[:self.rows].contiguous()
        seg = torch.zeros(E_loc + 1, dtype=torch.int64, device=flat.device)
        seg[1:] = torch.cumsum(pad2[r], 0)
        seg = seg.clamp(max=self.rows)                                        # (a no-op without a capacity)
        self.seg_off = seg.int()
        self.counts = torch.minimum(counts.view(W, E_loc)[r], seg[1:] - seg[:-1]).int().contiguous()
        self.T, self.k = T, k


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, plan: _Plan, ep: EPContext):
        from ..ops import kernels as K
        T, D = x.shape
        ws = ep.workspace("tok", T, D)
        ws.tensor.view(T, D).copy_(x)
        ep.barrier.wait()
        xp = torch.empty((plan.rows, D), dtype=torch.bfloat16, device=x.device)
        K.moe_zero_pad(xp, plan.seg_off, plan.counts)
        K.moe_pull_rows(ws.c_ptrs, ep.world, D, plan.src_rank, plan.src_row, xp)
        ctx.plan, ctx.ep, ctx.D = plan, ep, D
        return xp

    @staticmethod
    def backward(ctx, dxp):
        from ..ops import kernels as K
        plan, ep, D = ctx.plan, ctx.ep, ctx.D
        ws = ep.workspace("rows", plan.max_rows, D)
        ws.tensor.view(plan.max_rows, D)[:plan.rows].copy_(dxp)
        ep.barrier.wait()
        dx = K.moe_gather_sum_peer(ws.c_ptrs, ep.world, D, plan.dst_rank, plan.dst_pos, D)
        return dx, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, residual, plan: _Plan, ep: EPContext):
        from ..ops import kernels as K
        D = y.shape[1]
        ws = ep.workspace("rows", plan.max_rows, D)
        ws.tensor.view(plan.max_rows, D)[:plan.rows].copy_(y)
        ep.barrier.wait()
        out = K.moe_gather_sum_peer(ws.c_ptrs, ep.world, D, plan.dst_rank, plan.dst_pos, D, residual)
        ctx.plan, ctx.ep, ctx.D, ctx.has_res = plan, ep, D, residual is not None
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops import kernels as K
        plan, ep, D = ctx.plan, ctx.ep, ctx.D
        T = plan.T
        ws = ep.workspace("tok", T, D)
        ws.tensor.view(T, D).copy_(dout)
        ep.barrier.wait()
        dy = torch.empty((plan.rows, D), dtype=torch.bfloat16, device=dout.device)
        K.moe_zero_pad(dy, plan.seg_off, plan.counts)
        K.moe_pull_rows(ws.c_ptrs, ep.world, D, plan.src_rank, plan.src_row, dy)
        return dy, (dout if ctx.has_res else None), None, None


def _reference_local_share(layer, x_all, w_all, idx_all, first_expert: int, n_local: int):
    """sum over this rank's experts of w * expert(x) for ALL gathered tokens (plain PyTorch, any device)."""
    from ..ops import functional as F
    out = torch.zeros_like(x_all, dtype=torch.float32)
    kind = layer.cfg.activation
    for le in range(n_local):
        e = first_expert + le
        hit = idx_all == e                                      # [WT, k]
        rows = hit.any(-1).nonzero(as_tuple=True)[0]
        if rows.numel() == 0:
            continue
        xs = x_all[rows]
        wsum = (w_all[rows] * hit[rows].to(w_all.dtype)).sum(-1, keepdim=True)
        h = F.glu(xs @ layer.gate_proj[le].t(), xs @ layer.up_proj[le].t(), kind)
        out = out.index_add(0, rows, (wsum * (h @ layer.down_proj[le].t()).float()))
    return out


def expert_parallel_forward(layer, x: torch.Tensor, weights: torch.Tensor, idx: torch.Tensor, residual=None,
                            recompute: bool = False):
    """x [T, D] this rank's tokens; weights / idx [T, k] over ALL experts. Returns [T, D]. `recompute`: keep the
    dispatched rows and rebuild the experts' activations in backward on this rank (no second exchange)."""
    ep: EPContext = layer.ep
    W, r = ep.world, ep.rank
    E = layer.cfg.num_experts
    E_loc = E // W
    idx_all = _AllGather.apply(idx.int(), ep.group, W, r)
    w_all = _AllGather.apply(weights.float(), ep.group, W, r)
    D = x.shape[1]
    if not (ep.fused and x.dtype == torch.bfloat16 and D % 64 == 0 and layer.cfg.moe_hidden_dim % 64 == 0):
        x_all = _AllGather.apply(x, ep.group, W, r)
        share = _reference_local_share(layer, x_all, w_all, idx_all, r * E_loc, E_loc)
        y = _ReduceScatter.apply(share, ep.group, W, r).to(x.dtype)
        return y if residual is None else y + residual
    from ..ops import moe as moe_ops
    plan = _Plan(idx_all, E, ep)
    xp = _Dispatch.apply(x.contiguous(), plan, ep)
    # routing weight of every row this rank owns (slots owned elsewhere land in the spare entry, cut off again)
    wrow = torch.zeros(plan.rows + 1, dtype=torch.float32, device=x.device).index_put((plan.own_dest,),
                                                                                         w_all.reshape(-1))[:plan.rows]
    y = moe_ops.local_experts(xp, wrow, plan.seg_off, plan.counts, layer.gate_proj, layer.up_proj, layer.down_proj,
                              layer.cfg.activation, recompute=recompute)
    return _Combine.apply(y, residual, plan, ep)


def shard_experts(model, ep: EPContext):
    """Keep this rank's E / ep experts of every MoE layer. Expert parameters become rank-local (`dp_sharded`:
    their gradients already cover every token routed to them); all other parameters stay whole and have their
    gradients summed over the group by the trainer, since every rank trains on its own tokens."""
    from ..models.transformer import MoELayer
    W, r = ep.world, ep.rank
    with torch.no_grad():
        for mod in model.modules():
            if isinstance(mod, MoELayer):
                E = mod.cfg.num_experts
                if E % W:
                    raise ValueError(f"{E} experts do not divide over {W} ranks")
                n = E // W
                for name in ("gate_proj", "up_proj", "down_proj"):
                    p = getattr(mod, name)
                    q = nn.Parameter(p.data[r * n:(r + 1) * n].clone(), requires_grad=p.requires_grad)
                    q.dp_sharded = True
                    q.shard_spec = (0, r, W)
                    q.shard_group = ep.group
                    setattr(mod, name, q)
                mod.ep = ep
                mod.ep_group = ep.group if ep.group is not None else True
    model.dp_shard = ep      # the trainer sums the gradients of whole parameters over this group
    return model
