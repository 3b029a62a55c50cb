"""Which engine of a rollout group serves a trajectory (tunix/rl/rollout/rollout_traffic_router.py:15-36; the
reference ships the interface only). Two routers are provided: by stable hash of the trajectory id (the same
trajectory always meets the same engine and its prefix cache, in every process) and round robin."""
from __future__ import annotations

import abc
import dataclasses
import itertools

from ...experimental.worker.routing import stable_route_hash


@dataclasses.dataclass(kw_only=True)
class RolloutTrafficRoutingParams:
    trajectory_id: int


class RolloutTrafficRouter(abc.ABC):
    @abc.abstractmethod
    def route(self, params: RolloutTrafficRoutingParams) -> int:
        """The index of the rollout engine."""


class HashTrafficRouter(RolloutTrafficRouter):
    def __init__(self, num_engines: int):
        if num_engines <= 0:
            raise ValueError("num_engines must be positive")
        self.num_engines = num_engines

    def route(self, params: RolloutTrafficRoutingParams) -> int:
        return stable_route_hash(params.trajectory_id) % self.num_engines


class RoundRobinTrafficRouter(RolloutTrafficRouter):
    def __init__(self, num_engines: int):
        if num_engines <= 0:
            raise ValueError("num_engines must be positive")
        self.num_engines, self._next = num_engines, itertools.count()

    def route(self, params: RolloutTrafficRoutingParams) -> int:
        return next(self._next) % self.num_engines
