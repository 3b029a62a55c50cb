"""Trainer -> rollout weight transfer between ranks with different layouts.

Each parameter is described by the rectangle of the full matrix that a rank holds (`TensorSpec`: rows x cols
ranges in full coordinates; tensors with more than two dimensions are flattened after the first). A transfer
plan intersects the rectangle a destination rank wants with the rectangles the source ranks hold and yields 2-D
blocks; sources that hold the same data are picked round-robin by destination rank so that the pulls spread
over the NVLink ports.

Execution on GPUs with symmetric memory (`WeightReshard.run`): every source rank stages its tensors, cast to
bf16 and with LoRA adapters merged (`W + scale * B A`, one GEMM with a residual epilogue), in one symmetric
flat buffer; after a flag barrier every destination rank pulls its blocks with `tb_pull_blocks` (plain P2P
loads, `csrc/comm.cu`) straight into its parameters; a second barrier releases the staging buffers. Elsewhere
(CPU / gloo) the same plan runs as matched `send` / `recv` pairs.

KV-head replication for rollout tensor parallelism wider than the number of kv heads is a plan-level matter:
the destination's rectangle simply names the rows of the head it needs (`kv_rows_for`), and several
destinations may name the same rows.

Reference: tunix/rl/reshard.py:171-262 (`reshard_pytree`) and tunix/generate/utils.py:861-1005
(`transfer_state_with_mappings`: key mapping, kv-head repeat, dtype cast, tied lm_head sync).
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from ..parallel import symm


@dataclasses.dataclass(frozen=True)
class TensorSpec:
    full_shape: tuple            # (rows, cols) of the whole matrix
    rows: tuple                  # [r0, r1) held by this rank
    cols: tuple                  # [c0, c1) held by this rank

    @property
    def local_shape(self):
        return (self.rows[1] - self.rows[0], self.cols[1] - self.cols[0])


def _as2d(shape) -> tuple:
    shape = tuple(shape)
    if len(shape) == 1:
        return (1, shape[0])
    return (shape[0], int(np.prod(shape[1:])))


def spec_of(param: torch.Tensor) -> TensorSpec:
    """Spec of a parameter from the marks the parallel modules leave on it: `shard_spec = (dim, index, count)`
    (set by tensor / weight / expert sharding); unmarked parameters are whole."""
    r, c = _as2d(param.shape)
    ss = getattr(param, "shard_spec", None)
    if ss is None:
        return TensorSpec((r, c), (0, r), (0, c))
    dim, index, count = ss
    if dim == 0:
        return TensorSpec((r * count, c), (index * r, (index + 1) * r), (0, c))
    if param.dim() != 2:
        raise ValueError("column sharding is described for matrices only")
    return TensorSpec((r, c * count), (0, r), (index * c, (index + 1) * c))


def kv_rows_for(num_kv_heads: int, head_dim: int, tp: int, tp_rank: int) -> tuple:
    """Rows of a k / v projection that tensor-parallel rank `tp_rank` needs; with tp > kv heads, consecutive
    ranks share a head (tunix/generate/utils.py:1007-1019 repeats the heads instead)."""
    if tp <= num_kv_heads:
        per = num_kv_heads // tp
        return (tp_rank * per * head_dim, (tp_rank + 1) * per * head_dim)
    h = tp_rank * num_kv_heads // tp
    return (h * head_dim, (h + 1) * head_dim)


@dataclasses.dataclass
class Block:
    name: str
    src_rank: int
    dst_rank: int
    src_rc: tuple        # (row0, col0) inside the source's local tensor
    dst_rc: tuple        # (row0, col0) inside the destination's local tensor
    rows: int
    cols: int


def plan_blocks(name: str, dst: TensorSpec, dst_rank: int, sources: Sequence[tuple]) -> list:
    """sources: [(rank, TensorSpec)]. Covers dst's rectangle with pieces of the sources' rectangles."""
    if not sources:
        raise KeyError(f"no source holds {name}")
    need = [(dst.rows[0], dst.rows[1], dst.cols[0], dst.cols[1])]
    out = []
    order = list(sources)
    k = dst_rank % len(order)
    order = order[k:] + order[:k]
    for rank, s in order:
        nxt = []
        for (r0, r1, c0, c1) in need:
            ir0, ir1 = max(r0, s.rows[0]), min(r1, s.rows[1])
            ic0, ic1 = max(c0, s.cols[0]), min(c1, s.cols[1])
            if ir0 >= ir1 or ic0 >= ic1:
                nxt.append((r0, r1, c0, c1))
                continue
            out.append(Block(name, rank, dst_rank, (ir0 - s.rows[0], ic0 - s.cols[0]), (ir0 - dst.rows[0], ic0 - dst.cols[0]),
                             ir1 - ir0, ic1 - ic0))
            # what is left of this rectangle: up to four strips around the intersection
            if r0 < ir0:
                nxt.append((r0, ir0, c0, c1))
            if ir1 < r1:
                nxt.append((ir1, r1, c0, c1))
            if c0 < ic0:
                nxt.append((ir0, ir1, c0, ic0))
            if ic1 < c1:
                nxt.append((ir0, ir1, ic1, c1))
        need = nxt
        if not need:
            break
    if need:
        raise ValueError(f"{name}: region {need[0]} is held by no source rank")
    return out


_BLOCK_DT = np.dtype([("src_off", "<i8"), ("dst_off", "<i8"), ("src_ld", "<i8"), ("dst_ld", "<i8"), ("src_rank", "<i4"),
                      ("rows", "<i4"), ("cols", "<i4"), ("pad", "<i4")])


def merged_weight(module) -> torch.Tensor:
    """Base weight of a Linear with its LoRA adapter folded in: W + scale * B A (bf16)."""
    w = module.base_weight()
    if getattr(module, "lora_a", None) is None or not getattr(module, "lora_enabled", True):
        return w
    a, b = module.lora_a, module.lora_b            # [r, in], [out, r]
    if w.is_cuda and w.dtype == torch.bfloat16 and a.shape[0] % 8 == 0:
        from ..ops import kernels as K
        return K.gemm(b, a, b_mn=True, residual=w.contiguous(), alpha=float(module.lora_scale))
    return (w.float() + module.lora_scale * (b.float() @ a.float())).to(w.dtype)


class WeightReshard:
    """Collective object: every rank of `group` constructs it with its own role.

    src_tensors: {name: tensor} this rank offers (empty on pure rollout ranks); dst_tensors: {name: tensor} this
    rank wants filled (empty on pure trainer ranks); specs default to `spec_of`. `key_map(dst_name) -> src_name`
    translates names (e.g. a tied lm_head that reads the embedding)."""

    def __init__(self, src_tensors: dict, dst_tensors: dict, *, group=None, src_specs: Optional[dict] = None,
                 dst_specs: Optional[dict] = None, key_map: Optional[Callable[[str], str]] = None, device=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.src, self.dst = dict(src_tensors), dict(dst_tensors)
        self.src_specs = {n: (src_specs or {}).get(n) or spec_of(t) for n, t in self.src.items()}
        self.dst_specs = {n: (dst_specs or {}).get(n) or spec_of(t) for n, t in self.dst.items()}
        self.key_map = key_map or (lambda n: n)
        any_t = next(iter({**self.src, **self.dst}.values()), None)
        self.device = torch.device(device) if device is not None else (any_t.device if any_t is not None else torch.device("cpu"))
        # every rank learns what every rank offers
        offers = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(offers, self.src_specs, group=group)
        else:
            offers = [self.src_specs]
        self.offers = offers
        # staging layout of each source rank: tensors in name order, 8-element aligned
        self.stage_off = []
        for specs in offers:
            off, table = 0, {}
            for n in sorted(specs):
                table[n] = off
                r, c = specs[n].local_shape
                off += (r * c + 7) // 8 * 8
            self.stage_off.append((table, off))
        self.blocks = []
        for n, spec in self.dst_specs.items():
            sn = self.key_map(n)
            srcs = [(r, offers[r][sn]) for r in range(self.world) if sn in offers[r]]
            self.blocks += plan_blocks(n, spec, self.rank, srcs)
        self.fused = self.world > 1 and self.device.type == "cuda" and symm.symm_available(group)
        self._stage = None
        self._barrier = None
        self._tables = None

    # ------------------------------------------------------------------------------------------ GPU path
    def _setup_fused(self):
        size = max(off for _, off in self.stage_off)
        self._stage = symm.symm_empty(max(size, 8), torch.bfloat16, self.device, self.group, zero=False)
        self._barrier = symm.SymmBarrier(self.device, self.group)
        tables = {}
        for b in self.blocks:
            sn = self.key_map(b.name)
            s_spec = self.offers[b.src_rank][sn]
            s_ld = s_spec.local_shape[1]
            d_ld = self.dst_specs[b.name].local_shape[1]
            if b.cols % 8 or s_ld % 8 or d_ld % 8 or b.src_rc[1] % 8 or b.dst_rc[1] % 8:
                raise ValueError(f"{b.name}: the P2P path moves 16-byte vectors; column extents must be multiples of 8")
            rec = (self.stage_off[b.src_rank][0][sn] + b.src_rc[0] * s_ld + b.src_rc[1], b.dst_rc[0] * d_ld + b.dst_rc[1],
                   s_ld, d_ld, b.src_rank, b.rows, b.cols, 0)
            tables.setdefault(b.name, []).append(rec)
        self._tables = {n: torch.from_numpy(np.array(v, dtype=_BLOCK_DT).view(np.uint8).reshape(-1)).to(self.device)
                        for n, v in tables.items()}
        self._nblocks = {n: len(v) for n, v in tables.items()}

    def _run_fused(self):
        from .. import _lib
        _lib.register_cuda_sigs({"tb_pull_blocks": [_lib.P, _lib.I, _lib.P, _lib.I, _lib.P, _lib.P]})
        if self._stage is None:
            self._setup_fused()
        table, _ = self.stage_off[self.rank]
        flat = self._stage.tensor
        for n, t in self.src.items():
            flat[table[n]:table[n] + t.numel()].view(t.shape).copy_(t)       # casts to bf16
        self._barrier.wait()
        for n, t in self.dst.items():
            if n not in self._tables:
                continue
            target = t if (t.dtype == torch.bfloat16 and t.is_contiguous()) else torch.empty(t.shape, dtype=torch.bfloat16,
                                                                                            device=t.device)
            rc = _lib.cuda().tb_pull_blocks(self._stage.c_ptrs, self.world, self._tables[n].data_ptr(), self._nblocks[n],
                                            target.data_ptr(), _lib.stream_ptr())
            _lib.check(rc, "tb_pull_blocks")
            if target is not t:
                t.copy_(target)
        self._barrier.wait()

    # ---------------------------------------------------------------------------------- send / recv path
    def _run_p2p(self):
        plans = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(plans, [dataclasses.astuple(b) for b in self.blocks], group=self.group)
        else:
            plans = [[dataclasses.astuple(b) for b in self.blocks]]
        for plan in plans:
            for (name, src_rank, dst_rank, src_rc, dst_rc, rows, cols) in plan:
                sn = self.key_map(name)
                if self.rank == src_rank:
                    s = self.src[sn]
                    piece = s.reshape(_as2d(s.shape))[src_rc[0]:src_rc[0] + rows, src_rc[1]:src_rc[1] + cols].contiguous()
                if self.rank == dst_rank:
                    d = self.dst[name]
                    view = d.view(_as2d(d.shape))[dst_rc[0]:dst_rc[0] + rows, dst_rc[1]:dst_rc[1] + cols]
                if src_rank == dst_rank:
                    if self.rank == src_rank:
                        view.copy_(piece)
                    continue
                if self.rank == src_rank:
                    dist.send(piece.to(torch.float32), dst=dist.get_global_rank(self.group, dst_rank) if self.group else dst_rank,
                              group=self.group)
                elif self.rank == dst_rank:
                    buf = torch.empty((rows, cols), dtype=torch.float32, device=d.device)
                    dist.recv(buf, src=dist.get_global_rank(self.group, src_rank) if self.group else src_rank, group=self.group)
                    view.copy_(buf)

    @torch.no_grad()
    def run(self) -> None:
        """Collective: fills every destination tensor from the current values of the source tensors."""
        if self.fused:
            self._run_fused()
        else:
            self._run_p2p()

    @property
    def bytes_pulled(self) -> int:
        return sum(b.rows * b.cols * 2 for b in self.blocks if b.src_rank != self.rank)


def model_sources(model, merge_lora: bool = True) -> dict:
    """{name: tensor} a trainer offers: parameters by name, Linear weights with LoRA merged when asked."""
    out = {}
    merged = {}
    if merge_lora:
        for mn, mod in model.named_modules():
            if getattr(mod, "lora_a", None) is not None:
                w = merged_weight(mod)
                w.shard_spec = getattr(mod.weight, "shard_spec", None)
                merged[f"{mn}.weight"] = w
    for n, p in model.named_parameters():
        if "lora_" in n and merge_lora:
            continue
        out[n] = merged.get(n, p.detach())
        if n in merged:
            continue
        if getattr(p, "shard_spec", None) is not None:
            out[n].shard_spec = p.shard_spec
    return out
