"""Where each role of an RL job runs, and how ranks that host different roles talk to each other.

The reference runs one controller process that owns every device; `ClusterConfig.role_to_mesh` gives each role
(actor, critic, reference, reward, rollout) a mesh, equal meshes mean "colocated", different ones
"disaggregated", and the controller simply calls into whichever mesh holds the model
(tunix/common/configs.py:476-517, tunix/rl/rl_cluster.py:196-287, tunix/cli/base_rl_pipeline.py:135-270).

Here there is one process per GPU, so the same two ideas become:

* `RolePlacement`: role -> set of ranks (from a `parallel.mesh.Mesh`, a list of ranks, or nothing = every
  rank), the process group of each set, the parallel strategy its mesh axes ask for (`fsdp` -> sharded
  optimizer / weight sharding, `tp` -> tensor parallelism), and the layout this amounts to.
* `RoleExchange`: the ranks that run the training loop ("controllers": the actor's ranks) hand work items to the
  ranks that host another role and get the results back, in rounds that every rank of the job joins. A rank
  that hosts no part of the loop (a pure rollout or reference rank) sits in `serve()` and answers rounds until
  it is told to stop. When a role lives on exactly the controllers' ranks, a call is a plain local call with no
  communication at all, which is the colocated layout.

A round is two collectives on host objects (token ids, log-prob arrays: small), so it runs on a gloo group
beside the NCCL one; tensors that are large (the weights) never go through it: they move peer to peer with
`rl/reshard.py`.

`begin()` and `end()` split a round so that the controllers can train on batch k while the rollout ranks
generate batch k+1 (the reference's asynchronous rollout when the meshes differ,
tunix/rl/rl_learner.py:151-156); rounds do not nest: a `begin` is followed by its `end` before the next.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Optional, Sequence

import torch.distributed as dist

from ..common.datatypes import Role
from ..parallel.mesh import Mesh


def _as_role(r) -> Role:
    return r if isinstance(r, Role) else Role(str(r))


class RolePlacement:
    def __init__(self, role_to_mesh: Optional[dict] = None, *, world: Optional[int] = None, rank: Optional[int] = None,
                 make_groups: bool = True):
        self.world = world if world is not None else (dist.get_world_size() if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank() if dist.is_initialized() else 0)
        everyone = list(range(self.world))
        self.meshes: dict = {}
        self._ranks: dict = {}
        for role, m in (role_to_mesh or {}).items():
            role = _as_role(role)
            if isinstance(m, Mesh):
                self.meshes[role] = m
                self._ranks[role] = sorted(int(r) for r in m.devices.reshape(-1))
            elif m is None:
                self._ranks[role] = everyone
            else:
                self._ranks[role] = sorted(int(r) for r in m)
            bad = [r for r in self._ranks[role] if not 0 <= r < self.world]
            if bad or not self._ranks[role]:
                raise ValueError(f"role {role}: ranks {bad or '[]'} are not part of a job of {self.world} ranks")
        self._groups: dict = {}
        self.host_group = None
        if make_groups and dist.is_initialized() and self.world > 1:
            # every rank creates every group, in one order
            for key in sorted({tuple(v) for v in self._ranks.values()}):
                if list(key) != everyone and len(key) > 1:
                    self._groups[key] = dist.new_group(list(key))
            if "gloo" not in str(dist.get_backend()):
                self.host_group = dist.new_group(everyone, backend="gloo")

    # ------------------------------------------------------------------ queries
    def ranks(self, role) -> list:
        return self._ranks.get(_as_role(role), list(range(self.world)))

    def has(self, role, rank: Optional[int] = None) -> bool:
        return (self.rank if rank is None else rank) in self.ranks(role)

    def same(self, a, b) -> bool:
        return self.ranks(a) == self.ranks(b)

    def group(self, role):
        """Process group over the role's ranks; None means the default (world) group, also for one-rank roles."""
        return self._groups.get(tuple(self.ranks(role)))

    def index(self, role, rank: Optional[int] = None) -> int:
        return self.ranks(role).index(self.rank if rank is None else rank)

    def axis_size(self, role, axis: str) -> int:
        m = self.meshes.get(_as_role(role))
        if m is None:
            return len(self.ranks(role)) if axis == "fsdp" else 1      # a bare rank list is data parallel
        return m.axis_size(axis)

    def axis_group(self, role, axis: str):
        m = self.meshes.get(_as_role(role))
        if m is None:
            return self.group(role)
        return m.group(axis)

    def replica_groups(self, role) -> list:
        """The role's ranks as groups that each hold ONE copy of the model: the ranks along the `tp` axis of its mesh
        form a group (they work on the same items together), everything else multiplies the copies."""
        m = self.meshes.get(_as_role(role))
        if m is None or m.axis_size("tp") <= 1:
            return [[r] for r in self.ranks(role)]
        import numpy as np
        ax = m.axis_names.index("tp")
        lines = np.moveaxis(m.devices, ax, -1).reshape(-1, m.shape[ax])
        return sorted([int(r) for r in line] for line in lines)

    @property
    def controllers(self) -> list:
        return self.ranks(Role.ACTOR)

    @property
    def is_controller(self) -> bool:
        return self.rank in self.controllers

    @property
    def layout(self) -> str:
        """"colocated": every placed role sits on the actor's ranks; "disaggregated": the rollout ranks and the
        actor's ranks are disjoint; "mixed": anything else."""
        if all(self.same(r, Role.ACTOR) for r in self._ranks):
            return "colocated"
        if not set(self.controllers) & set(self.ranks(Role.ROLLOUT)):
            return "disaggregated"
        return "mixed"

    def describe(self) -> dict:
        return {str(r): self.ranks(r) for r in Role} | {"layout": self.layout}


def split_evenly(n: int, parts: int) -> list:
    """[(start, stop)] of `parts` contiguous chunks of range(n) whose sizes differ by at most one."""
    base, extra = divmod(n, parts)
    out, s = [], 0
    for i in range(parts):
        e = s + base + (1 if i < extra else 0)
        out.append((s, e))
        s = e
    return out


@dataclasses.dataclass
class _Round:
    role: Any
    op: str
    mine: list                 # (submitter rank, index in its list, item) this rank executes
    counts: list               # items submitted per rank
    results: Optional[list] = None
    local: bool = False
    report: bool = True        # False on the non-leading ranks of a model-parallel group: the leader reports the results


class RoleExchange:
    """Rounds of work between controllers and the ranks of other roles.

    handlers: {(Role, op): fn(list of items) -> list of results}, registered on the ranks that host the role.
    Special rounds: `sync` runs `on_sync()` on every rank (the weight transfer is itself a collective);
    `stop` ends `serve()`."""

    def __init__(self, placement: RolePlacement, on_sync: Optional[Callable[[], None]] = None):
        self.p = placement
        self.handlers: dict = {}
        self.on_sync = on_sync
        self._open: Optional[_Round] = None
        self.rounds = 0

    def register(self, role, op: str, fn: Callable[[list], list]) -> None:
        self.handlers[(_as_role(role), op)] = fn

    # ------------------------------------------------------------------ plumbing
    def _gather(self, obj) -> list:
        if self.p.world == 1 or not dist.is_initialized():
            return [obj]
        out = [None] * self.p.world
        dist.all_gather_object(out, obj, group=self.p.host_group)
        return out

    def is_local(self, role) -> bool:
        """The role sits on exactly the controllers' ranks: every controller serves its own items, no round."""
        return self.p.ranks(role) == self.p.controllers

    def _assign(self, role, submitted: list) -> tuple:
        flat = [(r, i, it) for r, items in enumerate(submitted) for i, it in enumerate(items or [])]
        groups = self.p.replica_groups(role)          # every rank of a group gets the group's share
        mine, report = [], True
        for gi, g in enumerate(groups):
            if self.p.rank in g:
                s, e = split_evenly(len(flat), len(groups))[gi]
                mine, report = flat[s:e], g[0] == self.p.rank
        return mine, [len(items or []) for items in submitted], report

    # -------------------------------------------------------------------- rounds
    def begin(self, role, op: str, items: Sequence) -> _Round:
        """Controllers: hand `items` to the ranks of `role`. Returns the round to pass to `end`."""
        if self._open is not None:
            raise RuntimeError("a round is already open: rounds do not nest")
        role = _as_role(role)
        if self.is_local(role):
            rd = _Round(role, op, [(self.p.rank, i, it) for i, it in enumerate(items)], [], local=True)
        else:
            submitted = self._gather(("work", str(role), op, list(items)))
            mine, counts, report = self._assign(role, [s[3] if s and s[0] == "work" else [] for s in submitted])
            rd = _Round(role, op, mine, counts, report=report)
        self._open = rd
        return rd

    def _execute(self, rd: _Round) -> None:
        if rd.results is not None:
            return
        if not rd.mine:
            rd.results = []
            return
        fn = self.handlers.get((rd.role, rd.op))
        if fn is None:
            raise KeyError(f"rank {self.p.rank} hosts {rd.role} but has no handler for {rd.op!r}")
        out = fn([it for _, _, it in rd.mine])
        if len(out) != len(rd.mine):
            raise ValueError(f"handler {rd.op!r} returned {len(out)} results for {len(rd.mine)} items")
        rd.results = list(out)

    def end(self, rd: _Round) -> list:
        """Results for the items this rank submitted, in order."""
        if self._open is not rd:
            raise RuntimeError("end() of a round that is not the open one")
        self._execute(rd)          # a controller that also hosts the role works here
        self._open = None
        self.rounds += 1
        if rd.local:
            return rd.results
        tagged = [(r, i, res) for (r, i, _), res in zip(rd.mine, rd.results)] if rd.report else []
        everything = self._gather(tagged)
        mine = [None] * (rd.counts[self.p.rank] if self.p.rank < len(rd.counts) else 0)
        for chunk in everything:
            for r, i, res in chunk or []:
                if r == self.p.rank:
                    mine[i] = res
        return mine

    def call(self, role, op: str, items: Sequence) -> list:
        return self.end(self.begin(role, op, items))

    def sync(self) -> None:
        """Controllers: run the weight transfer on every rank of the job."""
        if self._open is not None:
            raise RuntimeError("a round is open")
        if self.p.world > 1 and not all(self.is_local(r) for r in self.p._ranks):
            self._gather(("sync",))
        if self.on_sync is not None:
            self.on_sync()

    def stop(self) -> None:
        """Controllers: release the ranks that sit in `serve()`."""
        if self.p.world > 1 and not all(self.is_local(r) for r in self.p._ranks):
            self._gather(("stop",))

    # ------------------------------------------------------------------- workers
    def serve(self) -> int:
        """Ranks outside the training loop: answer rounds until `stop`. Returns the number of rounds served."""
        if self.p.is_controller:
            raise RuntimeError("controllers run the training loop, not serve()")
        served = 0
        while True:
            submitted = self._gather(None)
            head = next((s for s in submitted if s), None)
            if head is None or head[0] == "stop":
                return served
            if head[0] == "sync":
                if self.on_sync is not None:
                    self.on_sync()
                continue
            _, role, op, _ = head
            role = _as_role(role)
            mine, counts, report = self._assign(role, [s[3] if s and s[0] == "work" else [] for s in submitted])
            rd = _Round(role, op, mine, counts, report=report)
            self._execute(rd)
            self._gather([(r, i, res) for (r, i, _), res in zip(rd.mine, rd.results)] if report else [])
            served += 1
