"""Public configuration dataclasses (field names follow tunix/common/configs.py).

TrainingConfig :327-390, RLTrainingConfig :393-473, RolloutConfig :72-280, RLProfileConfig :283-311,
ClusterConfig :477-517, CacheConfig (tunix/generate/sampler.py). Engine-specific vLLM / SGLang
knobs of the reference map onto the options of the in-house paged engine
(`page_size`, `max_running_requests`, `max_num_batched_tokens`, `hbm_utilization`,
`chunked_prefill_size`, `deterministic_sampling`, `free_kv_during_sync`).
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Optional, Tuple


@dataclasses.dataclass
class MetricsLoggerOptions:
    log_dir: Optional[str] = None
    flush_every_n_steps: int = 100
    project_name: str = "tunix_b200"
    run_name: str = ""
    backend_factories: Optional[list] = None   # callables returning LoggingBackend objects
    use_tensorboard: bool = True
    use_wandb: bool = False
    use_jsonl: bool = True
    enable_opentelemetry: bool = False         # also write every scalar as an OpenTelemetry gauge


@dataclasses.dataclass
class ProfilerOptions:
    log_dir: str = ""
    skip_first_n_steps: int = 1
    profiler_steps: int = 1
    set_profile_options: bool = False


@dataclasses.dataclass
class PerfMetricsOptions:
    enable_perf_v1: bool = True
    enable_perf_v2: bool = False
    log_dir: Optional[str] = None
    enable_trace_writer: bool = False
    custom_export_fn: Any = None


@dataclasses.dataclass
class CheckpointingOptions:
    """Save every >=180 s by default, keep the latest 3, async (tunix/sft/checkpoint_options.py:103-111)."""
    save_interval_steps: Optional[int] = None
    save_interval_secs: Optional[float] = 180.0
    max_to_keep: Optional[int] = 3
    enable_async_checkpointing: bool = True
    timeout_secs: int = 1200

    @staticmethod
    def from_dict(d: dict | None) -> "CheckpointingOptions":
        if d is None:
            return CheckpointingOptions()
        known = {f.name for f in dataclasses.fields(CheckpointingOptions)}
        bad = set(d) - known
        if bad:
            raise ValueError(f"unknown checkpointing options: {sorted(bad)}")
        opts = CheckpointingOptions(**d)
        if opts.save_interval_steps is not None:
            opts.save_interval_secs = None
        return opts


@dataclasses.dataclass(kw_only=True)
class TrainingConfig:
    eval_every_n_steps: int
    max_steps: Optional[int] = None
    gradient_accumulation_steps: Optional[int] = None
    checkpoint_root_directory: Optional[str] = None
    checkpointing_options: Any = None
    resume_from_checkpoint_on_init: bool = True
    metrics_logging_options: Optional[MetricsLoggerOptions] = None
    profiler_options: Optional[ProfilerOptions] = None
    perf_metrics_options: Optional[PerfMetricsOptions] = None
    data_sharding_axis: Tuple[str, ...] = ("fsdp",)
    max_inflight_computations: int = 2
    metrics_prefix: str = ""
    pbar_description: Optional[str] = "Training"
    max_seq_token_per_tpu: Optional[int] = None       # packing token budget per row
    max_segments_per_packed_row: Optional[int] = None
    # multi-rank jobs: a rank whose heartbeat has been silent this long makes every other rank leave `train()` with
    # `parallel.watchdog.RankFailure` before its next step, instead of waiting in a collective (None = no watchdog)
    rank_failure_timeout_s: Optional[float] = None

    @property
    def sequence_packing_enabled(self) -> bool:
        return is_sequence_packing_enabled(self)

    def get_with_default(self, key: str, default: Any) -> Any:
        val = getattr(self, key)
        return default if val is None else val


def is_sequence_packing_enabled(config: Any) -> bool:
    budget = getattr(config, "max_seq_token_per_tpu", None)
    return isinstance(budget, int) and budget > 0


@dataclasses.dataclass(kw_only=True)
class RLProfileConfig:
    start_invocation: int = 2
    num_invocations: int = 1
    output_dir: str = ""
    timeout_secs: float = 60.0

    def __post_init__(self):
        if self.start_invocation < 0:
            raise ValueError(f"start_invocation must be >= 0. Got: {self.start_invocation}")
        if self.num_invocations <= 0:
            raise ValueError(f"num_invocations must be > 0. Got: {self.num_invocations}")
        if math.isnan(self.timeout_secs) or self.timeout_secs <= 0:
            raise ValueError(f"timeout_secs must be > 0. Got: {self.timeout_secs}")


@dataclasses.dataclass(kw_only=True)
class RLTrainingConfig(TrainingConfig):
    actor_optimizer: Any = None
    critic_optimizer: Any = None
    mini_batch_size: Optional[int] = None
    train_micro_batch_size: Optional[int] = None
    rollout_micro_batch_size: Optional[int] = None
    compute_logps_micro_batch_size: Optional[int] = None
    compute_logps_chunk_size: int = 0
    rl_profiler_config: Optional[RLProfileConfig] = None

    def __post_init__(self):
        for name in ("mini_batch_size", "train_micro_batch_size", "rollout_micro_batch_size",
                     "compute_logps_micro_batch_size"):
            v = getattr(self, name)
            if v is not None and v <= 0:
                raise ValueError(f"{name} must be positive, got {v}")
        if self.compute_logps_chunk_size < 0:
            raise ValueError("compute_logps_chunk_size must be >= 0")
        if self.mini_batch_size is not None:
            if self.train_micro_batch_size is None:
                self.train_micro_batch_size = self.mini_batch_size
            if self.mini_batch_size % self.train_micro_batch_size != 0:
                raise ValueError(
                    f"mini_batch_size ({self.mini_batch_size}) must be divisible by train_micro_batch_size "
                    f"({self.train_micro_batch_size})")
            derived = self.mini_batch_size // self.train_micro_batch_size
            if self.gradient_accumulation_steps is not None and self.gradient_accumulation_steps != derived:
                raise ValueError("gradient_accumulation_steps is derived from mini/micro batch sizes in RL training")
            self.gradient_accumulation_steps = derived
        if self.rollout_micro_batch_size is None:
            self.rollout_micro_batch_size = self.train_micro_batch_size
        if self.compute_logps_micro_batch_size is None:
            self.compute_logps_micro_batch_size = self.train_micro_batch_size


@dataclasses.dataclass
class CacheConfig:
    cache_size: int
    num_layers: int
    num_kv_heads: int
    head_dim: int


@dataclasses.dataclass(kw_only=True)
class RolloutConfig:
    max_tokens_to_generate: int = 64
    temperature: float = 0.9
    top_p: Optional[float] = 1.0
    top_k: Optional[int] = None
    seed: Optional[int] = None
    max_prompt_length: int = 64
    kv_cache_size: int = 1024
    data_type: Any = None
    eos_tokens: Optional[list] = None
    rollout_mapping_config: Any = None
    tensor_parallel_size: int = -1
    data_parallel_size: int = -1
    expert_parallel_size: int = 1
    return_logprobs: bool = True
    return_routed_experts: bool = False
    store_routed_experts: bool = False
    partial_rollout: bool = False
    # in-house paged engine
    page_size: int = 64
    max_running_requests: int = 256
    max_num_batched_tokens: int = 8192
    hbm_utilization: float = 0.3
    chunked_prefill_size: int = 4096
    deterministic_sampling: bool = True
    free_kv_during_sync: bool = False
    use_cuda_graph: bool = True


@dataclasses.dataclass(kw_only=True)
class ClusterConfig:
    role_to_mesh: dict
    role_to_logical_axis_rule: Optional[dict] = None
    rollout_engine: Any = "vanilla"
    offload_to_cpu: bool = False
    gc_collect_after_weight_sync: bool = True
    shard_frozen_models: bool = True   # an `fsdp` axis on a frozen role's mesh stores it as gathered-on-use row blocks
    training_config: RLTrainingConfig = None
    rollout_config: Any = None   # RolloutConfig or {Mode: RolloutConfig}
