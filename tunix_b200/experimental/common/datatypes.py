"""Control-plane data types of the distributed RL stack (tunix/experimental/common/datatypes.py:105-165 and the
request / response DTOs around it). Plain dataclasses: they travel through `torch.distributed` object
collectives or any pickling transport."""
from __future__ import annotations

import dataclasses
import enum
import time
from typing import Any, Optional


class WorkerState(str, enum.Enum):
    CREATED = "created"
    INITIALIZING = "initializing"
    COMPILING = "compiling"        # building native libraries / capturing graphs
    READY = "ready"
    BUSY = "busy"
    SYNCING = "syncing"            # weight synchronisation in progress
    DRAINING = "draining"
    STOPPED = "stopped"
    FAILED = "failed"


ALLOWED_TRANSITIONS = {
    WorkerState.CREATED: {WorkerState.INITIALIZING, WorkerState.FAILED, WorkerState.STOPPED},
    WorkerState.INITIALIZING: {WorkerState.COMPILING, WorkerState.READY, WorkerState.FAILED},
    WorkerState.COMPILING: {WorkerState.READY, WorkerState.FAILED},
    WorkerState.READY: {WorkerState.BUSY, WorkerState.SYNCING, WorkerState.DRAINING, WorkerState.FAILED},
    WorkerState.BUSY: {WorkerState.READY, WorkerState.DRAINING, WorkerState.FAILED},
    WorkerState.SYNCING: {WorkerState.READY, WorkerState.FAILED},
    WorkerState.DRAINING: {WorkerState.STOPPED, WorkerState.FAILED},
    WorkerState.STOPPED: set(),
    WorkerState.FAILED: {WorkerState.STOPPED},
}


class IllegalTransition(RuntimeError):
    pass


def check_transition(old: WorkerState, new: WorkerState) -> None:
    if new not in ALLOWED_TRANSITIONS[old]:
        raise IllegalTransition(f"{old.value} -> {new.value} is not an allowed worker transition")


@dataclasses.dataclass
class HealthReport:
    worker_id: str
    state: WorkerState
    timestamp: float = dataclasses.field(default_factory=time.time)
    policy_version: int = 0
    inflight: int = 0
    detail: str = ""


class Role(str, enum.Enum):
    """Roles of the models in an RL job (tunix/experimental/common/datatypes.py, `Role`)."""
    ACTOR = "actor"
    CRITIC = "critic"
    REFERENCE = "reference"
    REWARD = "reward"
    ROLLOUT = "rollout"


def role_name(role) -> str:
    return role.value if isinstance(role, enum.Enum) else str(role)


@dataclasses.dataclass(frozen=True)
class GenerationArgs:
    """Sampling settings of a dispatch; a field left None falls back to the request's own default."""
    max_tokens: Optional[int] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    seed: Optional[int] = None

    def as_kwargs(self) -> dict:
        return {k: v for k, v in dataclasses.asdict(self).items() if v is not None}


@dataclasses.dataclass
class RolloutRequest:
    request_id: str
    prompt_token_ids: list
    group_id: Optional[str] = None
    max_tokens: int = 256
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: Optional[int] = None
    seed: Optional[int] = None
    policy_version: int = 0
    metadata: dict = dataclasses.field(default_factory=dict)


@dataclasses.dataclass
class RolloutResponse:
    request_id: str
    tokens: list
    logprobs: Optional[list] = None
    text: Optional[str] = None
    policy_version: int = 0
    finish_reason: str = "stop"
    group_id: Optional[str] = None
    metadata: dict = dataclasses.field(default_factory=dict)


@dataclasses.dataclass
class RLTrainerPayload:
    """One training example on its way from scoring to the trainer, with its lineage."""
    example: Any
    policy_version: int
    group_id: Optional[str] = None
    reward: Optional[float] = None
    created_at: float = dataclasses.field(default_factory=time.time)
