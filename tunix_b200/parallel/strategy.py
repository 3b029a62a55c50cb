"""From a named mesh to the parallel form of a model and its optimizer.

The reference annotates every weight with mesh axes and lets GSPMD act on them (`fsdp`, `tp`,
tunix/models/llama3/model.py:47-82; the mesh comes from the CLI's `model_config.mesh`,
tunix/cli/config.py). Here the axes select one of the explicit strategies of this package:

    ('fsdp',)            size N     whole bf16 weights, sharded fp32 master / moments (`parallel/fsdp.py`, ZeRO-2),
                                    or with `shard_weights` weights stored as row blocks that the GEMMs gather
                                    (`parallel/fsdp3.py`, ZeRO-3)
    ('tp',)              size T     tensor parallel with sequence-parallel activations (`parallel/tp.py`)
    ('fsdp', 'tp')       N x T      tensor parallel inside each group of T adjacent ranks; the N groups are data
                                    parallel replicas whose gradients are summed over the `fsdp` axis before the
                                    update (optimizer state is not sharded in this combination)
    ('sp',) / ('fsdp', 'sp')        context parallel over `sp` (`parallel/cp.py`: every rank of an `sp` group keeps
                                    a slice of the sequence axis, attention gathers K / V over the group); the
                                    weights are whole on every rank and the optimizer is ZeRO-2 over all ranks

`apply_parallelism` is what the CLI entry points and `RLCluster` call; it returns the (possibly new) optimizer and
a short description for logs.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch
import torch.distributed as dist


@dataclasses.dataclass
class ParallelPlan:
    kind: str                      # single | zero2 | zero3 | tp | dp_tp | sp
    fsdp: int = 1
    tp: int = 1
    sp: int = 1
    dp_group: object = None        # gradients are summed over it before the update (dp_tp only)

    def describe(self) -> str:
        return {"single": "single rank", "zero2": f"zero2 over {self.fsdp} ranks", "zero3": f"zero3 over {self.fsdp} ranks",
                "tp": f"tp{self.tp}", "dp_tp": f"dp{self.fsdp} x tp{self.tp}",
                "sp": f"zero2 over {self.fsdp * self.sp} ranks, sequence over {self.sp}"}[self.kind]


def plan_for(mesh, shard_weights: bool = False) -> ParallelPlan:
    if mesh is None or mesh.size <= 1:
        return ParallelPlan("single")
    fsdp, tp, sp = mesh.axis_size("fsdp"), mesh.axis_size("tp"), mesh.axis_size("sp")
    other = [n for n in mesh.axis_names if n not in ("fsdp", "tp", "sp") and mesh.axis_size(n) > 1]
    if other:
        raise ValueError(f"mesh axes {other} have no strategy here; use 'fsdp', 'tp' and / or 'sp'")
    if sp > 1:
        if tp > 1 or shard_weights:
            raise ValueError("context parallelism ('sp') combines with 'fsdp' (zero2) only")
        return ParallelPlan("sp", fsdp, 1, sp)
    if tp > 1 and fsdp > 1:
        if shard_weights:
            raise ValueError("weight sharding (zero3) and tensor parallelism are not combined; drop one of them")
        return ParallelPlan("dp_tp", fsdp, tp)
    if tp > 1:
        return ParallelPlan("tp", 1, tp)
    return ParallelPlan("zero3" if shard_weights else "zero2", fsdp, 1)


def apply_parallelism(model, optimizer, mesh, shard_weights: bool = False, device=None):
    """-> (optimizer, plan). Slices / shards `model` in place as the plan says. Every rank of the mesh calls it."""
    plan = plan_for(mesh, shard_weights)
    if plan.kind == "single" or not dist.is_initialized():
        return optimizer, plan
    device = device or next(model.parameters()).device
    if plan.kind == "sp":
        from . import cp, fsdp
        cp.apply_context_parallel(model, mesh.group("sp"))
        if optimizer is not None:
            comm = "p2p" if torch.device(device).type == "cuda" else "nccl"
            optimizer = fsdp.shard_optimizer(optimizer, mesh.all_group(), comm=comm)
    elif plan.tp > 1:
        from . import tp as tp_lib
        tp_lib.apply_tensor_parallel(model, tp_lib.TPContext(group=mesh.group("tp"), device=device))
        if plan.kind == "dp_tp":
            plan.dp_group = mesh.group("fsdp")
            model.dp_replica_group = plan.dp_group      # the trainer sums gradients over it before the update
    elif plan.kind == "zero3":
        from . import fsdp3
        fsdp3.apply_weight_sharding(model, fsdp3.CommContext(group=mesh.group("fsdp"), device=device))
    elif plan.kind == "zero2" and optimizer is not None:
        from . import fsdp
        comm = "p2p" if torch.device(device).type == "cuda" else "nccl"
        optimizer = fsdp.shard_optimizer(optimizer, mesh.group("fsdp"), comm=comm)
    return optimizer, plan


def sum_replica_grads(model, optimizer) -> None:
    """dp x tp: add up the gradient buffers of the data-parallel replicas (one all-reduce over the flat buffer)."""
    group = getattr(model, "dp_replica_group", None)
    if group is None or dist.get_world_size(group) <= 1:
        return
    optimizer.buffers.collect_autograd_grads()
    dist.all_reduce(optimizer.buffers.grad_flat, group=group)
