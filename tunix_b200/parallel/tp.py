"""Tensor parallelism with sequence-parallel activations, on GEMMs that carry their collective.

Between tensor-parallel regions the residual stream is sharded over the tp ranks along the flattened token
dimension (rank r holds rows [r, r+1) * M / tp). A column-parallel projection all-gathers its input and a
row-parallel projection reduce-scatters its output; both collectives run INSIDE the GEMM kernel
(`csrc/gemm.cu`: copier / reducer CTAs next to the tcgen05 tile CTAs, data over NVLink peer memory):

    column forward   y[M, N/tp]   = gather(x_s) @ W_c^T            all-gather -> GEMM   (mode 1)
    column backward  dx_s         = scatter_sum(dy @ W_c)          GEMM -> reduce-scatter
                     dW_c         = dy^T @ gather(x_s)             all-gather (contraction) -> GEMM (mode 3)
    row forward      y_s[M/tp, N] = scatter_sum(x @ W_r^T) + res_s GEMM -> reduce-scatter
    row backward     dx           = gather(dy_s) @ W_r             all-gather -> GEMM   (mode 1)
                     dW_r         = gather(dy_s)^T @ x             plain GEMM on the buffer just gathered

Every fused call is preceded by the device-side flag barrier of `symm.SymmBarrier`: it makes the peers'
shards (or the previous reader's end) visible before remote memory is touched. Without symmetric memory
(CPU / gloo, one rank) the same functions run `torch.distributed` collectives around plain matmuls, which is
what the CPU tests exercise.

Reference: the reference expresses this through GSPMD sharding annotations (`act_btd = (fsdp, None, tp)`,
`ffw_weight_df = (fsdp, tp)`, tunix/models/llama3/model.py:47-82) and lets XLA insert the collectives.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import symm


class TPContext:
    """Process group + symmetric workspaces of one tensor-parallel group."""

    def __init__(self, group=None, device=None, n_aux: int = 0):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.n_aux = n_aux
        self.fused = self.world > 1 and self.device.type == "cuda" and symm.symm_available(group)
        self.barrier = symm.SymmBarrier(self.device, group) if self.fused else None
        self._gather: dict = {}
        self._partial: dict = {}

    # ------------------------------------------------------------ workspaces (collective on first use)
    def gather_ws(self, rows: int, cols: int):
        """Two symmetric buffers per shape, used alternately: a rank refills its rows of buffer i while a slower
        peer may still be reading buffer i-1; by the time buffer i comes round again every peer has passed the
        barrier of the call in between, so nobody reads it any more."""
        key = (rows, cols)
        pair = self._gather.get(key)
        if pair is None:
            pair = {"n": 0, "ws": []}
            for _ in range(2):
                buf = symm.symm_empty(rows * cols, torch.bfloat16, self.device, self.group, zero=True)
                pair["ws"].append({"buf": buf, "epoch": 0,
                                   "ready": torch.zeros(rows // 128 + 1, dtype=torch.int32, device=self.device)})
            self._gather[key] = pair
        pair["n"] += 1
        return pair["ws"][pair["n"] & 1]

    def partial_ws(self, M: int, N: int):
        key = (M, N)
        ws = self._partial.get(key)
        if ws is None:
            ws = {"part": symm.symm_empty(M * N, torch.bfloat16, self.device, self.group, zero=True),
                  "done": symm.symm_empty(M // 128 + 1, torch.int32, self.device, self.group, zero=True),
                  "total": ctypes.c_uint(0), "work": torch.zeros(1, dtype=torch.int32, device=self.device)}
            self._partial[key] = ws
        return ws

    def fusable(self, M: int, *dims: int) -> bool:
        return self.fused and M % (128 * self.world) == 0 and all(d % 64 == 0 for d in dims)

    # ----------------------------------------------------------------------------------- primitives
    def all_gather_rows(self, x_s: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x_s
        out = torch.empty((x_s.shape[0] * self.world, *x_s.shape[1:]), dtype=x_s.dtype, device=x_s.device)
        dist.all_gather_into_tensor(out, x_s.contiguous(), group=self.group)
        return out

    def reduce_scatter_rows(self, y: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return y
        m = y.shape[0] // self.world
        if "nccl" in str(dist.get_backend(self.group)):
            out = torch.empty((m, *y.shape[1:]), dtype=y.dtype, device=y.device)
            dist.reduce_scatter_tensor(out, y.contiguous(), group=self.group)
            return out
        y = y.float().contiguous()       # gloo has no reduce-scatter
        dist.all_reduce(y, group=self.group)
        return y[self.rank * m:(self.rank + 1) * m]

    def ag_gemm(self, x_s: torch.Tensor, w: torch.Tensor, *, w_mn: bool = False, bias=None):
        """gather(x_s) @ op(w)^T. x_s [M/tp, K]; w [N, K] (or [K, N] when w_mn). Returns (y [M, N], gathered x)."""
        from ..ops import kernels as K
        m, Kd = x_s.shape
        M = m * self.world
        N = w.shape[1] if w_mn else w.shape[0]
        if not self.fusable(M, Kd):
            xg = self.all_gather_rows(x_s)
            y = xg @ (w if w_mn else w.t())
            return (y if bias is None else y + bias), xg
        ws = self.gather_ws(M, Kd)
        buf = ws["buf"]
        xg = buf.tensor.view(M, Kd)
        xg[self.rank * m:(self.rank + 1) * m].copy_(x_s)
        self.barrier.wait()
        ws["epoch"] += 1
        y = torch.empty((M, N), dtype=torch.bfloat16, device=x_s.device)
        K.gemm_ag(buf.c_ptrs, self.rank, self.world, 1, M, Kd, w, y, M, N, Kd, ws["ready"], ws["epoch"], other_mn=w_mn,
                  bias=bias, n_aux=self.n_aux)
        return y, xg

    def ag_wgrad(self, dy: torch.Tensor, x_s: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False):
        """dy^T @ gather(x_s): dy [M, N] local in full, x_s [M/tp, K] -> [N, K] (bf16, or into `out`)."""
        from ..ops import kernels as K
        m, Kd = x_s.shape
        M, N = dy.shape
        if not self.fusable(M, Kd, N):
            xg = self.all_gather_rows(x_s)
            g = dy.t().float() @ xg.float()
            if out is None:
                return g.to(dy.dtype)
            return out.add_(g.to(out.dtype)) if accumulate else out.copy_(g)
        ws = self.gather_ws(M, Kd)
        buf = ws["buf"]
        buf.tensor.view(M, Kd)[self.rank * m:(self.rank + 1) * m].copy_(x_s)
        self.barrier.wait()
        ws["epoch"] += 1
        if out is None:
            out = torch.empty((N, Kd), dtype=torch.bfloat16, device=dy.device)
        K.gemm_ag(buf.c_ptrs, self.rank, self.world, 3, M, Kd, dy, out, N, Kd, M, ws["ready"], ws["epoch"],
                  other_mn=True, accumulate=accumulate, n_aux=self.n_aux)
        return out

    # ---- weights sharded by rows over the group (ZeRO-3 style data parallelism, parallel/fsdp3.py)
    def gemm_gather_w(self, x: torch.Tensor, w_s: torch.Tensor, bias=None, residual=None) -> torch.Tensor:
        """x @ gather_rows(w_s)^T: x [M, K] local, w_s [N/W, K] this rank's rows of the weight (mode 2)."""
        from ..ops import kernels as K
        n, Kd = w_s.shape
        N, M = n * self.world, x.shape[0]
        if not self.fusable(N, Kd):
            y = x @ self.all_gather_rows(w_s).t()
            y = y if bias is None else y + bias
            return y if residual is None else y + residual
        ws = self.gather_ws(N, Kd)
        buf = ws["buf"]
        buf.tensor.view(N, Kd)[self.rank * n:(self.rank + 1) * n].copy_(w_s)
        self.barrier.wait()
        ws["epoch"] += 1
        y = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        K.gemm_ag(buf.c_ptrs, self.rank, self.world, 2, N, Kd, x, y, M, N, Kd, ws["ready"], ws["epoch"], bias=bias,
                  residual=residual, n_aux=self.n_aux)
        return y

    def gemm_gather_w_t(self, dy: torch.Tensor, w_s: torch.Tensor) -> torch.Tensor:
        """dy @ gather_rows(w_s): dy [M, N], w_s [N/W, K] -> [M, K]; the gathered rows are the contraction (mode 3)."""
        from ..ops import kernels as K
        n, Kd = w_s.shape
        N, M = n * self.world, dy.shape[0]
        if not self.fusable(N, Kd):
            return dy @ self.all_gather_rows(w_s)
        ws = self.gather_ws(N, Kd)
        buf = ws["buf"]
        buf.tensor.view(N, Kd)[self.rank * n:(self.rank + 1) * n].copy_(w_s)
        self.barrier.wait()
        ws["epoch"] += 1
        dx = torch.empty((M, Kd), dtype=torch.bfloat16, device=dy.device)
        K.gemm_ag(buf.c_ptrs, self.rank, self.world, 3, N, Kd, dy, dx, M, Kd, N, ws["ready"], ws["epoch"], n_aux=self.n_aux)
        return dx

    def wgrad_scatter(self, dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        """scatter_sum_rows(dy^T @ x): dy [M, N], x [M, K] (this rank's tokens) -> [N/W, K] summed over ranks."""
        from ..ops import kernels as K
        M, N = dy.shape
        Kd = x.shape[1]
        if not self.fusable(N, Kd) or M % 8:
            return self.reduce_scatter_rows((dy.t().float() @ x.float()).to(dy.dtype)).to(dy.dtype)
        ws = self.partial_ws(N, Kd)
        self.barrier.wait()
        out = torch.empty((N // self.world, Kd), dtype=torch.bfloat16, device=dy.device)
        K.gemm_rs(dy, x, ws["part"].c_ptrs, ws["done"].c_ptrs, out, ws["total"], ws["work"], self.rank, self.world, N, Kd, M,
                  a_mn=True, b_mn=True, n_aux=self.n_aux)
        return out

    def gemm_rs(self, x: torch.Tensor, w: torch.Tensor, *, w_mn: bool = False, residual_s=None) -> torch.Tensor:
        """scatter_sum(x @ op(w)^T) (+ residual_s). x [M, K_local]; returns [M/tp, N]."""
        from ..ops import kernels as K
        M, Kd = x.shape
        N = w.shape[1] if w_mn else w.shape[0]
        if not self.fusable(M, N) or Kd % 8:
            y = self.reduce_scatter_rows(x @ (w if w_mn else w.t())).to(x.dtype)
            return y if residual_s is None else y + residual_s
        ws = self.partial_ws(M, N)
        self.barrier.wait()
        out = torch.empty((M // self.world, N), dtype=torch.bfloat16, device=x.device)
        K.gemm_rs(x, w, ws["part"].c_ptrs, ws["done"].c_ptrs, out, ws["total"], ws["work"], self.rank, self.world, M, N, Kd, b_mn=w_mn,
                  residual=residual_s.contiguous() if residual_s is not None else None, n_aux=self.n_aux)
        return out


def _wgrad_into(w_ref, compute):
    """Weight gradient either accumulated into `w_ref.main_grad` (fp32 flat buffer) or returned."""
    mg = getattr(w_ref, "main_grad", None)
    if mg is not None:
        compute(mg, True)
        w_ref.grad_added_to_main_grad = True
        for part in getattr(w_ref, "_joint_parts", ()):      # a joint view over several parameters' slots
            part.grad_added_to_main_grad = True
        return None
    return compute(None, False)


class _ColumnSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_s, w, bias, tp: TPContext):
        y, _ = tp.ag_gemm(x_s, w, bias=bias)
        ctx.save_for_backward(x_s, w)
        ctx.tp, ctx.w_ref, ctx.has_bias = tp, w, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x_s, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        dx = tp.gemm_rs(dy, w, w_mn=True) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            dw = _wgrad_into(ctx.w_ref, lambda out, acc: tp.ag_wgrad(dy, x_s, out, acc))
        db = dy.float().sum(0).to(dy.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db, None


class _RowSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, residual_s, tp: TPContext):
        y_s = tp.gemm_rs(x, w, residual_s=residual_s)
        ctx.save_for_backward(x, w)
        ctx.tp, ctx.w_ref, ctx.has_res = tp, w, residual_s is not None
        return y_s

    @staticmethod
    def backward(ctx, dy_s):
        from ..ops import kernels as K
        x, w = ctx.saved_tensors
        tp = ctx.tp
        dy_s = dy_s.contiguous()
        dx, dyg = tp.ag_gemm(dy_s, w, w_mn=True)            # [M, K_local]; dyg = gathered dy [M, N]
        dw = None
        if ctx.needs_input_grad[1]:
            def compute(out, acc):
                if x.is_cuda and x.dtype == torch.bfloat16:
                    return K.gemm(dyg, x, a_mn=True, b_mn=True, out=out, accumulate=acc) if out is not None else \
                        K.gemm(dyg, x, a_mn=True, b_mn=True)
                g = dyg.t().float() @ x.float()
                if out is None:
                    return g.to(x.dtype)
                return out.add_(g.to(out.dtype)) if acc else out.copy_(g)
            dw = _wgrad_into(ctx.w_ref, compute)
        return dx, dw, (dy_s if ctx.has_res else None), None


class _GatherTokens(torch.autograd.Function):
    """[M/tp, ...] token shard -> all [M, ...] tokens; backward sums the ranks' gradients and keeps the own shard."""

    @staticmethod
    def forward(ctx, x_s, tp: TPContext):
        ctx.tp = tp
        return tp.all_gather_rows(x_s)

    @staticmethod
    def backward(ctx, g):
        return ctx.tp.reduce_scatter_rows(g.contiguous()).to(g.dtype), None


class _ScatterSumTokens(torch.autograd.Function):
    """Partial sums [M, ...] on every rank -> this rank's token shard of their sum; backward gathers."""

    @staticmethod
    def forward(ctx, y, tp: TPContext):
        ctx.tp = tp
        return tp.reduce_scatter_rows(y.contiguous()).to(y.dtype)

    @staticmethod
    def backward(ctx, g):
        return ctx.tp.all_gather_rows(g.contiguous()), None


def gather_tokens(x_s, tp: TPContext):
    """Sequence-parallel shard [B/tp, ...] -> [B, ...] as a plain collective (the path for projections that carry
    adapters or a quantised base, whose GEMMs do not gather for themselves)."""
    return _GatherTokens.apply(x_s, tp) if tp.world > 1 else x_s


def scatter_sum_tokens(y, tp: TPContext):
    """Row-parallel partial outputs [B, ...] -> [B/tp, ...] summed over the group."""
    return _ScatterSumTokens.apply(y, tp) if tp.world > 1 else y


def column_parallel_linear(x_s, w, bias, tp: TPContext):
    """x_s [..., K] sharded over tokens -> [tp * rows, N_local] for all tokens, this rank's output features."""
    lead = x_s.shape[:-1]
    y = _ColumnSP.apply(x_s.reshape(-1, x_s.shape[-1]), w, bias, tp)
    return y.view(lead[0] * tp.world, *lead[1:], w.shape[0]) if len(lead) > 1 else y


def row_parallel_linear(x, w, residual_s, tp: TPContext):
    """x [..., K_local] for all tokens -> [rows / tp, N] token shard, summed over ranks (+ residual shard)."""
    lead = x.shape[:-1]
    r2 = residual_s.reshape(-1, residual_s.shape[-1]) if residual_s is not None else None
    y = _RowSP.apply(x.reshape(-1, x.shape[-1]), w, r2, tp)
    return y.view(lead[0] // tp.world, *lead[1:], w.shape[0]) if len(lead) > 1 else y


# ------------------------------------------------------------------------------------ model surgery
def shard_rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.shape[0] // world
    return t[rank * n:(rank + 1) * n].clone()


def shard_cols(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.shape[1] // world
    return t[:, rank * n:(rank + 1) * n].clone()


def apply_tensor_parallel(model, tp: TPContext):
    """Slice a Transformer's attention and MLP weights for `tp` in place and switch it to the sequence-parallel
    forward (`Transformer.forward` consults `model.tp`). Heads and the MLP hidden dimension are split over the
    ranks (kv heads too: num_kv_heads must be divisible by tp); embeddings, norms and lm_head stay replicated
    and see this rank's token shard only, so their gradients are summed over the group by
    `allreduce_replicated_grads` before the optimizer step."""
    cfg = model.config
    W, r = tp.world, tp.rank
    if cfg.num_heads % W or cfg.num_kv_heads % W or cfg.hidden_dim % W:
        raise ValueError(f"heads {cfg.num_heads}/{cfg.num_kv_heads} and hidden {cfg.hidden_dim} must divide by tp={W}")
    if cfg.is_moe:
        raise NotImplementedError("MoE layers use expert parallelism (parallel/ep.py), not tensor parallelism")
    with torch.no_grad():
        for layer in model.layers:
            at, mlp = layer.self_attn, layer.mlp
            for lin in (at.q_proj, at.k_proj, at.v_proj, mlp.gate_proj, mlp.up_proj):
                lin.weight = nn.Parameter(shard_rows(lin.weight.data, r, W), requires_grad=lin.weight.requires_grad)
                lin.weight.shard_spec = (0, r, W)
                lin.weight.shard_group = tp.group
                if lin.bias is not None:
                    lin.bias = nn.Parameter(shard_rows(lin.bias.data, r, W), requires_grad=lin.bias.requires_grad)
                    lin.bias.shard_spec = (0, r, W)
                    lin.bias.shard_group = tp.group
                lin.tp, lin.tp_mode = tp, "column"
                if lin.lora_b is not None:         # adapters attached before the split: B follows the output rows
                    lin.lora_b = nn.Parameter(shard_rows(lin.lora_b.data, r, W), requires_grad=lin.lora_b.requires_grad)
                    lin.lora_b.shard_spec, lin.lora_b.shard_group = (0, r, W), tp.group
            for lin in (at.o_proj, mlp.down_proj):
                lin.weight = nn.Parameter(shard_cols(lin.weight.data, r, W), requires_grad=lin.weight.requires_grad)
                lin.weight.shard_spec = (1, r, W)
                lin.weight.shard_group = tp.group
                lin.tp, lin.tp_mode = tp, "row"
                if lin.lora_a is not None:         # A follows the input columns
                    lin.lora_a = nn.Parameter(shard_cols(lin.lora_a.data, r, W), requires_grad=lin.lora_a.requires_grad)
                    lin.lora_a.shard_spec, lin.lora_a.shard_group = (1, r, W), tp.group
            if any(l.quant is not None for l in (at.q_proj, at.k_proj, at.v_proj, at.o_proj, mlp.gate_proj, mlp.up_proj,
                                                 mlp.down_proj)):
                raise NotImplementedError("quantise the base after the tensor-parallel split, not before")
    model.tp = tp
    mark_sharded_params(model)
    return model


def mark_sharded_params(model) -> None:
    """`p.tp_sharded`: True for parameters of which every rank holds a different slice. The rest is held in full by
    every rank and sees partial gradients (other tokens, or other output / input slices), which
    `allreduce_replicated_grads` sums. Of an adapter pair, the factor on the split side of its projection is
    sliced (B of a column-parallel projection, A of a row-parallel one) and the other one is replicated."""
    col, row = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj"), ("o_proj", "down_proj")
    for n, p in model.named_parameters():
        if n.endswith("lora_a"):
            p.tp_sharded = any(k in n for k in row)
        elif n.endswith("lora_b"):
            p.tp_sharded = any(k in n for k in col)
        else:
            p.tp_sharded = any(k in n for k in col + row)


def allreduce_replicated_grads(model, tp: TPContext) -> None:
    """Sum over the tp group the gradients of parameters every rank holds in full (they saw different tokens)."""
    if tp.world == 1:
        return
    from .fsdp3 import _coalesce_adjacent
    grads = []
    for p in model.parameters():
        if getattr(p, "tp_sharded", False):
            continue
        g = getattr(p, "main_grad", None)
        g = g if g is not None else p.grad
        if g is not None:
            grads.append(g)
    for g in _coalesce_adjacent(grads):          # neighbouring slots of the flat gradient buffer go in one collective
        dist.all_reduce(g, group=tp.group)


def grad_sumsq(model, tp: TPContext) -> torch.Tensor:
    """Squared global gradient norm: sliced parameters contribute once per rank (summed over the group),
    replicated ones once (their gradients are already identical on all ranks)."""
    dev = next(model.parameters()).device
    sharded = torch.zeros((), dtype=torch.float32, device=dev)
    repl = torch.zeros((), dtype=torch.float32, device=dev)
    for p in model.parameters():
        g = getattr(p, "main_grad", None)
        g = g if g is not None else p.grad
        if g is None:
            continue
        s = g.float().pow(2).sum()
        if getattr(p, "tp_sharded", False):
            sharded += s
        else:
            repl += s
    if tp.world > 1:
        dist.all_reduce(sharded, group=tp.group)
    return (sharded + repl).reshape(1)


def local_batch(model, t: Optional[torch.Tensor]):
    """This rank's slice of a batch-major tensor under sequence-parallel TP (identity without TP)."""
    tp = getattr(model, "tp", None)
    if tp is None or t is None or tp.world == 1:
        return t
    n = t.shape[0] // tp.world
    return t[tp.rank * n:(tp.rank + 1) * n]


# ---------------------------------------------------------------------------------- vocab-parallel lm_head
class _VocabParallelLogprobs(torch.autograd.Function):
    """log p(target) (and entropy) with the vocabulary rows of the head sharded over the group: every rank scores
    its slice in row chunks (fp32 logits of `chunk x V/tp` at a time), and the ranks exchange three numbers per
    token: the running maximum (all-reduce max), then sum exp(z - max), the target's logit and, for the entropy,
    sum exp(z - max) * z (all-reduce sum). The backward pass recomputes the chunk's logits and forms
    dz = (softmax - onehot) * g locally; dh is summed over the group, dW stays with the shard.
    (tunix/models/*: lm_head sharded `(fsdp, tp)`, tunix/models/llama3/model.py:47-82)."""

    @staticmethod
    def forward(ctx, h, w_shard, targets, tp, softcap, temperature, want_entropy, chunk):
        rows, D = h.shape
        Vs = w_shard.shape[0]
        lo = tp.rank * Vs
        t = targets.reshape(-1).long()
        local = (t >= lo) & (t < lo + Vs)
        m = torch.empty(rows, dtype=torch.float32, device=h.device)
        stats = torch.zeros(rows, 3, dtype=torch.float32, device=h.device)          # sumexp, target logit, sum exp*z

        def logits(s0, s1):
            z = (h[s0:s1].to(w_shard.dtype) @ w_shard.t()).float()
            if softcap > 0:
                z = softcap * torch.tanh(z / softcap)
            return z / temperature
        for s0 in range(0, rows, chunk):
            m[s0:s0 + chunk] = logits(s0, min(s0 + chunk, rows)).max(-1).values
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=tp.group)
        for s0 in range(0, rows, chunk):
            s1 = min(s0 + chunk, rows)
            z = logits(s0, s1)
            e = torch.exp(z - m[s0:s1, None])
            stats[s0:s1, 0] = e.sum(-1)
            idx = (t[s0:s1] - lo).clamp(0, Vs - 1)
            stats[s0:s1, 1] = torch.where(local[s0:s1], z.gather(1, idx[:, None])[:, 0], torch.zeros_like(m[s0:s1]))
            if want_entropy:
                stats[s0:s1, 2] = (e * z).sum(-1)
        dist.all_reduce(stats, group=tp.group)
        lse = m + torch.log(stats[:, 0])
        valid = t >= 0
        logp = torch.where(valid, stats[:, 1] - lse, torch.zeros_like(lse))
        ent = (lse - stats[:, 2] / stats[:, 0]) if want_entropy else None
        ctx.save_for_backward(h, w_shard, t, lse)
        ctx.tp, ctx.softcap, ctx.temperature, ctx.chunk, ctx.lo = tp, softcap, temperature, chunk, lo
        ctx.mark_non_differentiable(*([ent] if ent is not None else []))
        return (logp, ent) if want_entropy else (logp, None)

    @staticmethod
    def backward(ctx, g_logp, _g_ent):
        h, w, t, lse = ctx.saved_tensors
        tp, softcap, temp, chunk, lo = ctx.tp, ctx.softcap, ctx.temperature, ctx.chunk, ctx.lo
        rows, Vs = h.shape[0], w.shape[0]
        g = torch.where(t >= 0, g_logp.reshape(-1).float(), torch.zeros_like(lse))
        dh = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
        dw = torch.zeros(w.shape, dtype=torch.float32, device=h.device)
        local = (t >= lo) & (t < lo + Vs)
        for s0 in range(0, rows, chunk):
            s1 = min(s0 + chunk, rows)
            raw = (h[s0:s1].to(w.dtype) @ w.t()).float()
            z = (softcap * torch.tanh(raw / softcap) if softcap > 0 else raw) / temp
            dz = -torch.exp(z - lse[s0:s1, None])                                     # d logp / dz = onehot - softmax
            idx = (t[s0:s1] - lo).clamp(0, Vs - 1)
            dz.scatter_add_(1, idx[:, None], local[s0:s1, None].float())
            dz = dz * (g[s0:s1, None] / temp)
            if softcap > 0:
                dz = dz * (1.0 - torch.tanh(raw / softcap) ** 2)
            dh[s0:s1] = dz @ w.float()
            dw += dz.t() @ h[s0:s1].float()
        dist.all_reduce(dh, group=tp.group)
        return dh.to(h.dtype), dw.to(w.dtype), None, None, None, None, None, None


def vocab_parallel_logprobs(h, w_shard, targets, tp: TPContext, *, softcap: float = 0.0, temperature: float = 1.0,
                            want_entropy: bool = False, chunk: int = 2048):
    """Per-token log p(target) with the head's vocabulary rows sharded over `tp` (rank r holds rows
    [r * V/tp, (r+1) * V/tp)). `h` [..., D] and `targets` [...] are the same on every rank of the group; negative
    targets are ignored (log-prob 0). Returns (logp fp32, entropy fp32 | None), identical on all ranks."""
    h2 = h.reshape(-1, h.shape[-1])
    logp, ent = _VocabParallelLogprobs.apply(h2, w_shard, targets, tp, float(softcap or 0.0), float(temperature),
                                             bool(want_entropy), int(chunk) if chunk and chunk > 0 else 2048)
    return logp.view(targets.shape), (ent.view(targets.shape) if ent is not None else None)
