"""Typed trajectories in the Agent Trajectory Interchange Format, ATIF v1.7, with the RL extensions this framework
records (tunix/experimental/trajectory/trajectory.py:29-1555).

Base documents (`Step`, `TrajectoryMetadata`, `Trajectory` and the small records they hold) carry what any agent
framework can read: who said what, tool calls, observations, token counts. The RL subclasses (`TunixAgentStep`,
`TunixEnvStep`, `TunixTrajectoryMetadata`, `TunixTrajectory`) add token ids, loss masks, log-probs, policy versions,
rewards and routed experts. Projecting a subclass to base ATIF packs its extra fields under
`extra["_tunix_extensions"]` (arrays become lists), so a document stays valid ATIF for readers that do not know the
extensions and round-trips exactly for those that do; step ids are 0-based in memory and 1-based in ATIF.

Models are dataclasses with explicit JSON conversion: unknown keys are rejected (a typo must not vanish into a
document), `None` fields are left out of the output."""
from __future__ import annotations

import dataclasses
import datetime
import enum
from typing import Any, ClassVar, Dict, List, Optional, Sequence, Union

import numpy as np

ATIF_SCHEMA_VERSION = "ATIF-v1.7"
TUNIX_EXTENSIONS_KEY = "_tunix_extensions"


class Source(str, enum.Enum):
    SYSTEM = "system"
    USER = "user"
    AGENT = "agent"


def _jsonable(v: Any) -> Any:
    if isinstance(v, np.ndarray):
        return v.tolist()
    if isinstance(v, np.generic):
        return v.item()
    if isinstance(v, enum.Enum):
        return v.value
    if isinstance(v, datetime.datetime):
        return v.isoformat()
    if isinstance(v, _Model):
        return v.to_json()
    if isinstance(v, dict):
        return {str(k): _jsonable(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [_jsonable(x) for x in v]
    return v


class _Model:
    """Dataclass base: strict `from_json`, `to_json` without None, nested models named in `_NESTED`
    ({field: model class}; a list field holds a list of that model), `validate()` after construction."""
    _NESTED: ClassVar[Dict[str, Any]] = {}

    def __post_init__(self) -> None:
        self.validate()

    def validate(self) -> None:
        pass

    @classmethod
    def field_names(cls) -> list:
        return [f.name for f in dataclasses.fields(cls)]

    def to_json(self) -> dict:
        out = {}
        for name in self.field_names():
            v = getattr(self, name)
            if v is not None:
                out[name] = _jsonable(v)
        return out

    @classmethod
    def _nested(cls) -> dict:
        merged: dict = {}
        for base in reversed(cls.__mro__):
            merged.update(getattr(base, "_NESTED", {}) if "_NESTED" in vars(base) else {})
        return merged

    @classmethod
    def from_json(cls, data: dict):
        if isinstance(data, cls):
            return data
        unknown = set(data) - set(cls.field_names())
        if unknown:
            raise ValueError(f"{cls.__name__}: unknown field(s) {sorted(unknown)}")
        nested = cls._nested()
        kw = {}
        for k, v in data.items():
            sub = nested.get(k)
            if sub is not None and v is not None:
                v = [sub.from_json(x) for x in v] if isinstance(v, list) else sub.from_json(v)
            kw[k] = v
        return cls(**kw)

    def copy(self):
        return type(self).from_json(self.to_json())


@dataclasses.dataclass
class SubagentTrajectoryRef(_Model):
    trajectory_id: Optional[str] = None
    session_id: Optional[str] = None
    trajectory_path: Optional[str] = None
    extra: Optional[dict] = None

    def validate(self) -> None:
        if self.trajectory_id is None and self.trajectory_path is None:
            raise ValueError("SubagentTrajectoryRef must set either trajectory_id or trajectory_path.")


@dataclasses.dataclass
class ObservationResult(_Model):
    source_call_id: Optional[str] = None
    content: Optional[str] = None
    subagent_trajectory_ref: Optional[List[SubagentTrajectoryRef]] = None
    extra: Optional[dict] = None
    _NESTED = {"subagent_trajectory_ref": SubagentTrajectoryRef}


@dataclasses.dataclass
class Observation(_Model):
    results: List[ObservationResult] = dataclasses.field(default_factory=list)
    _NESTED = {"results": ObservationResult}


@dataclasses.dataclass
class Metrics(_Model):
    prompt_tokens: Optional[int] = None
    completion_tokens: Optional[int] = None
    cached_tokens: Optional[int] = None
    cost_usd: Optional[float] = None
    prompt_token_ids: Optional[List[int]] = None
    completion_token_ids: Optional[List[int]] = None
    logprobs: Optional[List[float]] = None
    extra: Optional[dict] = None


@dataclasses.dataclass
class FinalMetrics(_Model):
    total_prompt_tokens: Optional[int] = None
    total_completion_tokens: Optional[int] = None
    total_cached_tokens: Optional[int] = None
    total_cost_usd: Optional[float] = None
    total_steps: Optional[int] = None
    extra: Optional[dict] = None


@dataclasses.dataclass
class ToolCall(_Model):
    tool_call_id: str = ""
    function_name: str = ""
    arguments: dict = dataclasses.field(default_factory=dict)
    extra: Optional[dict] = None

    def validate(self) -> None:
        if not self.tool_call_id or not self.function_name:
            raise ValueError("ToolCall needs a tool_call_id and a function_name")
        if not isinstance(self.arguments, dict):
            raise ValueError("ToolCall.arguments must be a JSON object")


@dataclasses.dataclass
class Agent(_Model):
    name: str = ""
    version: str = ""
    model_name: Optional[str] = None
    tool_definitions: Optional[List[dict]] = None
    extra: Optional[dict] = None


_AGENT_ONLY = ("model_name", "reasoning_effort", "reasoning_content", "tool_calls", "metrics")
_LLM_ONLY = ("metrics", "reasoning_content", "model_name", "reasoning_effort")


def _base_of(cls, root):
    """Field names of `root` (the ATIF base) and the extension fields `cls` adds."""
    base = [f.name for f in dataclasses.fields(root)]
    return base, [n for n in cls.field_names() if n not in base]


def _pack(model: "_Model", root) -> Optional[dict]:
    """JSON of `model` projected onto `root`: extension fields move under extra[EXTENSIONS_KEY]. None when `model`
    already is a plain `root`."""
    if type(model) is root:
        return None
    base, ext = _base_of(type(model), root)
    data = {k: _jsonable(getattr(model, k)) for k in base if getattr(model, k) is not None}
    packed = {k: _jsonable(getattr(model, k)) for k in ext if getattr(model, k) is not None}
    if packed:
        extra = dict(data.get("extra") or {})
        extra[type(model).EXTENSIONS_KEY] = {**(extra.get(type(model).EXTENSIONS_KEY) or {}), **packed}
        data["extra"] = extra
    return data


def _unpack(base_model: "_Model", cls, root) -> dict:
    """JSON for `cls` from a base document: known extension fields move from extra[EXTENSIONS_KEY] to the top level;
    keys `cls` does not know stay where they are."""
    data = base_model.to_json()
    _, ext = _base_of(cls, root)
    extra = dict(data.get("extra") or {})
    packed = dict(extra.get(cls.EXTENSIONS_KEY) or {})
    for k in list(packed):
        if k in ext:
            data[k] = packed.pop(k)
    if packed:
        extra[cls.EXTENSIONS_KEY] = packed
    else:
        extra.pop(cls.EXTENSIONS_KEY, None)
    data["extra"] = extra or None
    if data["extra"] is None:
        data.pop("extra")
    return data


@dataclasses.dataclass
class Step(_Model):
    step_id: int = 0
    source: Source = Source.USER
    message: str = ""
    timestamp: Optional[str] = None
    model_name: Optional[str] = None
    reasoning_effort: Optional[Union[str, float]] = None
    reasoning_content: Optional[str] = None
    tool_calls: Optional[List[ToolCall]] = None
    observation: Optional[Observation] = None
    metrics: Optional[Metrics] = None
    is_copied_context: Optional[bool] = None
    llm_call_count: Optional[int] = None
    extra: Optional[dict] = None
    _NESTED = {"tool_calls": ToolCall, "observation": Observation, "metrics": Metrics}
    EXTENSIONS_KEY: ClassVar[str] = ""
    ATIF_STEP_OFFSET: ClassVar[int] = 0             # what `to_atif_step()` adds to the id by default

    def __init_subclass__(cls, **kw) -> None:
        super().__init_subclass__(**kw)
        if not isinstance(cls.EXTENSIONS_KEY, str) or not cls.EXTENSIONS_KEY:
            raise TypeError(f"{cls.__name__} must define a non-empty string 'EXTENSIONS_KEY' ClassVar.")

    def validate(self) -> None:
        self.source = Source(self.source)
        if self.llm_call_count is not None and self.llm_call_count < 0:
            raise ValueError("llm_call_count must be >= 0")
        if self.source != Source.AGENT:
            for f in _AGENT_ONLY:
                if getattr(self, f) is not None:
                    raise ValueError(f"Field '{f}' is only applicable when source is 'agent', but source is '{self.source.value}'")
        elif self.llm_call_count == 0:
            for f in _LLM_ONLY:
                if getattr(self, f) is not None:
                    raise ValueError(f"Field '{f}' must be absent when llm_call_count is 0 (deterministic dispatch on a "
                                     "'source: agent' step)")

    def to_atif_step(self, step_id_offset: int = 0) -> "Step":
        data = _pack(self, Step)
        if data is None:
            return self
        data["step_id"] = self.step_id + step_id_offset
        return Step.from_json(data)

    def to_atif_json(self) -> dict:
        """The JSON of `to_atif_step()` without building the intermediate object (the writers' hot path)."""
        data = _pack(self, Step)
        if data is None:
            return self.to_json()
        data["step_id"] = self.step_id + type(self).ATIF_STEP_OFFSET
        return data


def _int_array(v, name: str, ndim: int = 1) -> Optional[np.ndarray]:
    if v is None:
        return None
    a = np.asarray(v)
    if a.size == 0:
        a = a.reshape((0,) * ndim).astype(np.int64)
    if a.ndim != ndim or not np.issubdtype(a.dtype, np.integer):
        raise ValueError(f"{name} must be an integer array with {ndim} dimension(s), got shape {a.shape} dtype {a.dtype}")
    return a


def _float_array(v, name: str) -> Optional[np.ndarray]:
    if v is None:
        return None
    a = np.asarray(v, np.float32)
    if a.ndim != 1:
        raise ValueError(f"{name} must be a 1-D float array, got shape {a.shape}")
    return a


@dataclasses.dataclass
class TunixAgentStep(Step):
    """An agent turn with what training needs: the sampled token ids, their loss mask and log-probs, the weights'
    version, the discounted return, and (for MoE replay) the routed experts of the prefill this turn's call ran:
    `prefill_routed_experts` [T, layers, k] covers sequence positions [prefill_start, prefill_start + T), of which the
    first `prefill_num_context` rows are context before this turn's generation."""
    EXTENSIONS_KEY: ClassVar[str] = TUNIX_EXTENSIONS_KEY
    ATIF_STEP_OFFSET: ClassVar[int] = 1
    mc_return: Optional[float] = None
    assistant_tokens: Any = None
    assistant_masks: Any = None
    logprobs: Any = None
    policy_version: Optional[int] = None
    prefill_routed_experts: Any = None
    prefill_start: Optional[int] = None
    prefill_num_context: Optional[int] = None

    def validate(self) -> None:
        super().validate()
        if self.source != Source.AGENT:
            raise ValueError(f"TunixAgentStep is only applicable when source is 'agent', but source is '{self.source.value}'")
        self.assistant_tokens = _int_array(self.assistant_tokens, "assistant_tokens")
        self.assistant_masks = _int_array(self.assistant_masks, "assistant_masks")
        self.logprobs = _float_array(self.logprobs, "logprobs")
        self.prefill_routed_experts = _int_array(self.prefill_routed_experts, "prefill_routed_experts", 3)
        trio = (self.prefill_routed_experts, self.prefill_start, self.prefill_num_context)
        if any(x is not None for x in trio) and not all(x is not None for x in trio):
            raise ValueError("prefill_routed_experts, prefill_start, and prefill_num_context must be either all None or all set")
        if self.prefill_routed_experts is not None:
            if self.prefill_start < 0:
                raise ValueError(f"prefill_start must be >= 0, got {self.prefill_start}")
            if not 0 <= self.prefill_num_context <= len(self.prefill_routed_experts):
                raise ValueError(f"prefill_num_context must be in [0, {len(self.prefill_routed_experts)}], got {self.prefill_num_context}")

    def to_atif_step(self, step_id_offset: int = 1) -> Step:
        return super().to_atif_step(step_id_offset)

    @classmethod
    def from_atif_step(cls, step: Step, step_id_offset: int = 1) -> "TunixAgentStep":
        data = _unpack(step, cls, Step)
        data["step_id"] = step.step_id - step_id_offset
        return cls.from_json(data)


@dataclasses.dataclass
class TunixEnvStep(Step):
    """What the environment (or the user / system) said, with its reward, terminal flag and the tokens it added to the
    context (mask 0: attended to, not trained on)."""
    EXTENSIONS_KEY: ClassVar[str] = TUNIX_EXTENSIONS_KEY
    ATIF_STEP_OFFSET: ClassVar[int] = 1
    reward: Optional[float] = None
    done: Optional[bool] = None
    env_tokens: Any = None
    env_masks: Any = None

    def validate(self) -> None:
        super().validate()
        if self.source not in (Source.SYSTEM, Source.USER):
            raise ValueError(f"TunixEnvStep is only applicable when source is 'system' or 'user', but source is '{self.source.value}'")
        self.env_tokens = _int_array(self.env_tokens, "env_tokens")
        self.env_masks = _int_array(self.env_masks, "env_masks")

    def to_atif_step(self, step_id_offset: int = 1) -> Step:
        return super().to_atif_step(step_id_offset)

    @classmethod
    def from_atif_step(cls, step: Step, step_id_offset: int = 1) -> "TunixEnvStep":
        data = _unpack(step, cls, Step)
        data["step_id"] = step.step_id - step_id_offset
        return cls.from_json(data)


def upcast_atif_step(step: Step) -> Step:
    """The RL step class for a base ATIF step, by its source; RL steps pass through."""
    if isinstance(step, (TunixAgentStep, TunixEnvStep)):
        return step
    return (TunixAgentStep if Source(step.source) == Source.AGENT else TunixEnvStep).from_atif_step(step)


@dataclasses.dataclass
class TrajectoryMetadata(_Model):
    """Everything about a trajectory except its steps."""
    agent: Agent = None
    schema_version: str = ATIF_SCHEMA_VERSION
    session_id: Optional[str] = None
    trajectory_id: Optional[str] = None
    notes: Optional[str] = None
    final_metrics: Optional[FinalMetrics] = None
    continued_trajectory_ref: Optional[str] = None
    extra: Optional[dict] = None
    _NESTED = {"agent": Agent, "final_metrics": FinalMetrics}
    EXTENSIONS_KEY: ClassVar[str] = ""
    _SUBCLASSES: ClassVar[list] = []

    def __init_subclass__(cls, **kw) -> None:
        super().__init_subclass__(**kw)
        if any(b.__name__ == "Trajectory" for b in cls.__mro__[1:]) or cls.__name__ == "Trajectory":
            return                                  # full trajectories share the root fields but are not metadata classes
        if not isinstance(cls.EXTENSIONS_KEY, str) or not cls.EXTENSIONS_KEY:
            raise TypeError(f"{cls.__name__} must define a non-empty string 'EXTENSIONS_KEY' ClassVar.")
        TrajectoryMetadata._SUBCLASSES.append(cls)

    def validate(self) -> None:
        if self.agent is None:
            raise ValueError("TrajectoryMetadata needs an agent")
        if isinstance(self.agent, dict):
            self.agent = Agent.from_json(self.agent)

    @classmethod
    def metadata_field_names(cls) -> list:
        return [n for n in cls.field_names() if n not in ("steps", "subagent_trajectories")]

    def to_atif_metadata(self) -> "TrajectoryMetadata":
        if type(self) is TrajectoryMetadata:
            return self
        return TrajectoryMetadata.from_json(self.to_atif_json())

    def to_atif_json(self) -> dict:
        """Plain ATIF metadata as JSON (steps of a full trajectory are left out)."""
        if type(self) is TrajectoryMetadata:
            return self.to_json()
        meta_cls = next((c for c in type(self).__mro__ if c in TrajectoryMetadata._SUBCLASSES), None)
        base = [f.name for f in dataclasses.fields(TrajectoryMetadata)]
        data = {k: _jsonable(getattr(self, k)) for k in base if getattr(self, k) is not None}
        if meta_cls is not None:
            ext = [n for n in meta_cls.metadata_field_names() if n not in base]
            packed = {k: _jsonable(getattr(self, k)) for k in ext if getattr(self, k) is not None}
            if packed:
                extra = dict(data.get("extra") or {})
                extra[meta_cls.EXTENSIONS_KEY] = {**(extra.get(meta_cls.EXTENSIONS_KEY) or {}), **packed}
                data["extra"] = extra
        return data

    def get_extensions(self) -> dict:
        cls = self.resolve_subclass(self)
        packed = (self.extra or {}).get(getattr(cls, "EXTENSIONS_KEY", "") or "")
        return packed if isinstance(packed, dict) else {}

    @classmethod
    def resolve_subclass(cls, metadata: "TrajectoryMetadata"):
        """The metadata class a stored base document belongs to, from the keys packed in its `extra`: the narrowest
        registered class whose extension fields cover the packed keys (normal case, and classes that have since gained
        optional fields); failing that, the widest class all of whose fields are present (a field has since been
        removed; the unknown keys stay in `extra`). Ties go to `cls`."""
        for c in type(metadata).__mro__:
            if c in TrajectoryMetadata._SUBCLASSES:
                return c
        if not metadata.extra:
            return TrajectoryMetadata
        base = [f.name for f in dataclasses.fields(TrajectoryMetadata)]
        covers, covered = [], []
        for sub in TrajectoryMetadata._SUBCLASSES:
            packed = metadata.extra.get(sub.EXTENSIONS_KEY)
            if not isinstance(packed, dict) or not packed:
                continue
            fields = {n for n in sub.metadata_field_names() if n not in base}
            if packed.keys() <= fields:
                covers.append((len(fields), sub is not cls, sub))
            elif fields <= packed.keys():
                covered.append((len(fields), sub is cls, sub))
        if covers:
            return min(covers, key=lambda t: t[:2])[2]
        if covered:
            return max(covered, key=lambda t: t[:2])[2]
        return TrajectoryMetadata

    @classmethod
    def from_atif_metadata(cls, metadata: "TrajectoryMetadata"):
        if isinstance(metadata, cls):
            return metadata
        return cls.from_json(_unpack(metadata, cls, TrajectoryMetadata))

    def create_trajectory(self, steps: Optional[Sequence] = None, subagent_trajectories: Optional[Sequence] = None) -> "Trajectory":
        data = {n: getattr(self, n) for n in TrajectoryMetadata.field_names()}
        return Trajectory(**data, steps=list(steps or []), subagent_trajectories=list(subagent_trajectories) if subagent_trajectories else None)


@dataclasses.dataclass
class Trajectory(TrajectoryMetadata):
    steps: list = dataclasses.field(default_factory=list)
    subagent_trajectories: Optional[list] = None
    _NESTED = {"steps": Step}
    STEP_OFFSET: ClassVar[int] = 1                  # ids of the first step

    def validate(self) -> None:
        super().validate()
        for i, s in enumerate(self.steps):
            if s.step_id != i + self.STEP_OFFSET:
                raise ValueError(f"step ids must be consecutive from {self.STEP_OFFSET}: position {i} has step_id {s.step_id}")

    @classmethod
    def from_json(cls, data: dict):
        if isinstance(data, cls):
            return data
        data = dict(data)
        subs = data.pop("subagent_trajectories", None)
        out = super().from_json(data)
        if subs is not None:
            out.subagent_trajectories = [cls.from_json(x) for x in subs]
        return out

    def metadata(self) -> TrajectoryMetadata:
        return TrajectoryMetadata(**{n: getattr(self, n) for n in TrajectoryMetadata.field_names()})

    def to_atif_trajectory(self) -> "Trajectory":
        """A plain ATIF trajectory (1-based step ids, extensions packed), embedded subagent trajectories included."""
        meta = self.to_atif_metadata()
        steps = [s.to_atif_step() if type(s) is not Step else s for s in self.steps]
        subs = [t.to_atif_trajectory() for t in self.subagent_trajectories] if self.subagent_trajectories else None
        return Trajectory(**{n: getattr(meta, n) for n in TrajectoryMetadata.field_names()}, steps=steps, subagent_trajectories=subs)

    def compute_final_metrics(self) -> FinalMetrics:
        ms = [s.metrics for s in self.steps if s.metrics is not None]
        tot = lambda f: sum(getattr(m, f) or 0 for m in ms) if any(getattr(m, f) is not None for m in ms) else None
        return FinalMetrics(total_prompt_tokens=tot("prompt_tokens"), total_completion_tokens=tot("completion_tokens"),
                            total_cached_tokens=tot("cached_tokens"), total_cost_usd=tot("cost_usd"), total_steps=len(self.steps))


@dataclasses.dataclass
class TunixTrajectoryMetadata(TrajectoryMetadata):
    EXTENSIONS_KEY: ClassVar[str] = TUNIX_EXTENSIONS_KEY
    prompt_id: Optional[str] = None
    group_index: int = 0
    target_policy_versions: Optional[List[int]] = None
    status: Optional[str] = None
    total_reward: Optional[float] = None
    masked_out: Optional[bool] = None
    hyperparams: Optional[dict] = None
    env_time: Optional[dict] = None
    reward_time: Optional[dict] = None

    def create_trajectory(self, steps: Optional[Sequence] = None, subagent_trajectories: Optional[Sequence] = None) -> "TunixTrajectory":
        steps = [upcast_atif_step(s) for s in (steps or [])]
        subs = [TunixTrajectory.from_atif_trajectory(t) for t in subagent_trajectories] if subagent_trajectories else None
        data = {n: getattr(self, n) for n in TunixTrajectoryMetadata.field_names()}
        return TunixTrajectory(**data, steps=steps, subagent_trajectories=subs)


@dataclasses.dataclass
class TunixTrajectory(TunixTrajectoryMetadata, Trajectory):
    STEP_OFFSET: ClassVar[int] = 0

    @classmethod
    def metadata_field_names(cls) -> list:
        return TunixTrajectoryMetadata.field_names()

    @classmethod
    def from_atif_trajectory(cls, traj: Trajectory) -> "TunixTrajectory":
        if isinstance(traj, cls):
            return traj
        meta = TunixTrajectoryMetadata.from_atif_metadata(traj.metadata())
        return meta.create_trajectory(traj.steps, traj.subagent_trajectories)

    def metadata(self) -> TunixTrajectoryMetadata:
        return TunixTrajectoryMetadata(**{n: getattr(self, n) for n in TunixTrajectoryMetadata.field_names()})

    @classmethod
    def from_json(cls, data: dict):
        """Reads either form: a plain ATIF document (1-based ids, packed extensions) or this class's own JSON."""
        if isinstance(data, cls):
            return data
        first = (data.get("steps") or [{}])[0]
        own = any(k in data for k in ("prompt_id", "group_index", "status", "total_reward")) or first.get("step_id") == 0
        if not own:
            return cls.from_atif_trajectory(Trajectory.from_json(data))
        data = dict(data)
        steps = [(TunixAgentStep if Source(s["source"]) == Source.AGENT else TunixEnvStep).from_json(s) if isinstance(s, dict) else s
                 for s in data.pop("steps", [])]
        subs = data.pop("subagent_trajectories", None)
        meta = TunixTrajectoryMetadata.from_json(data)
        out = meta.create_trajectory(steps, None)
        if subs:
            out.subagent_trajectories = [cls.from_json(x) for x in subs]
        return out
