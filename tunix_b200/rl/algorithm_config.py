"""Algorithm configuration dataclasses (tunix/rl/algorithm_config.py:21-286, PPOConfig tunix/rl/ppo/ppo_learner.py:49-120,
DAPO / Dr.GRPO configs tunix/rl/grpo/dapo_learner.py:28-161, drgrpo_learner.py:28-39)."""
from __future__ import annotations

import dataclasses
from typing import Optional

from . import function_registry

_VARIANTS = ["grpo", "drgrpo", "gspo-token", "ppo", "dapo"]
_ESTIMATORS = ["grpo", "gae", "drgrpo", "rloo", "grpo-loo"]
_POLICY_LOSSES = ["grpo", "ppo"]
_AGG_MODES = ["token-mean", "sequence-mean-token-mean", "sequence-mean-token-scale", "seq-mean-token-sum",
              "sequence-mean-token-sum-norm"]


@dataclasses.dataclass(kw_only=True)
class AlgorithmConfig:
    algo_variant: str = "grpo"
    advantage_estimator: str = "grpo"
    policy_loss_fn: str = "grpo"
    reward_manager: str = "sequence-level"
    kl_clamp_value: Optional[float] = None
    reward_num_workers: int = 0
    reward_worker_timeout_seconds: float = 180.0
    temperature: Optional[float] = dataclasses.field(default=None, init=False)
    use_rollout_logps: bool = True
    exact_token_continuity: bool = True
    sampler_is: Optional[str] = None               # "token" | "sequence"
    sampler_is_threshold: Optional[float] = 2.0
    sampler_rs: Optional[str] = None               # "token" | "geometric"
    sampler_rs_min: Optional[float] = None
    sampler_rs_max: Optional[float] = None
    seq_logprob_error_threshold: Optional[float] = None

    def __post_init__(self):
        self.temperature = None
        if self.algo_variant not in _VARIANTS:
            raise ValueError(f"algo_variant must be one of {_VARIANTS}. Received: {self.algo_variant!r}")
        if self.advantage_estimator not in _ESTIMATORS and \
                self.advantage_estimator not in function_registry.list_advantage_estimators():
            raise ValueError(f"advantage_estimator must be one of {_ESTIMATORS} or registered in function_registry. "
                             f"Received: {self.advantage_estimator}")
        if self.policy_loss_fn not in _POLICY_LOSSES and self.policy_loss_fn not in function_registry.list_policy_loss_fns():
            raise ValueError(f"policy_loss_fn must be one of {_POLICY_LOSSES} or registered in function_registry. "
                             f"Received: {self.policy_loss_fn}")
        if self.reward_num_workers < -1:
            raise ValueError(f"reward_num_workers must be >= 0, or -1 for one worker per CPU. Received: {self.reward_num_workers}")
        if self.reward_worker_timeout_seconds <= 0:
            raise ValueError("reward_worker_timeout_seconds must be > 0")
        if self.sampler_is is not None and self.sampler_is not in ("token", "sequence"):
            raise ValueError("sampler_is must be None, 'token' or 'sequence'")
        if self.sampler_rs is not None and self.sampler_rs not in ("token", "geometric"):
            raise ValueError("sampler_rs must be None, 'token' or 'geometric'")
        if self.sampler_is is not None and (self.sampler_is_threshold is None or self.sampler_is_threshold <= 0):
            raise ValueError("sampler_is_threshold must be positive when sampler_is is set")
        if self.sampler_rs is not None and self.sampler_rs_min is None and self.sampler_rs_max is None:
            raise ValueError("sampler_rs needs sampler_rs_min and/or sampler_rs_max")


@dataclasses.dataclass(kw_only=True)
class GRPOConfig(AlgorithmConfig):
    loss_agg_mode: str = "sequence-mean-token-mean"
    loss_algo: str = "grpo"            # "grpo" | "gspo-token"
    num_generations: int = 2
    num_iterations: int = 1
    beta: float = 0.04
    kl_loss_mode: str = "kl"           # "kl" | "mse_kl" | "low_var_kl"
    epsilon: float = 0.2
    epsilon_high: Optional[float] = None
    epsilon_c: Optional[float] = None

    def __post_init__(self):
        super().__post_init__()
        if self.epsilon_high is None:
            self.epsilon_high = self.epsilon
        if self.num_generations <= 1 and self.advantage_estimator in ("grpo", "drgrpo", "rloo", "grpo-loo"):
            raise ValueError(f"num_generations must be > 1 for group-relative advantages. Received: {self.num_generations}")
        if self.loss_algo not in ("grpo", "gspo-token"):
            raise ValueError(f"loss_algo must be 'grpo' or 'gspo-token'. Received: {self.loss_algo}")
        if self.loss_agg_mode not in _AGG_MODES:
            raise ValueError(f"loss_agg_mode must be one of {_AGG_MODES}. Received: {self.loss_agg_mode}")
        if self.kl_loss_mode not in ("kl", "mse_kl", "low_var_kl"):
            raise ValueError(f"unknown kl_loss_mode {self.kl_loss_mode}")
        if self.epsilon_c is not None and self.epsilon_c <= 1.0:
            raise ValueError("epsilon_c (dual-clip) must be > 1")


@dataclasses.dataclass(kw_only=True)
class DAPOConfig(GRPOConfig):
    """beta = 0, clip-higher, token-mean aggregation, optional overlong-buffer reward shaping."""
    algo_variant: str = "dapo"
    beta: float = 0.0
    epsilon_high: Optional[float] = 0.28
    loss_agg_mode: str = "token-mean"
    overlong_buffer: Optional[dict] = None   # {"enable": bool, "overlong_buffer_length": int, "overlong_buffer_penalty": float, "max_response_length": int}


@dataclasses.dataclass(kw_only=True)
class DrGRPOConfig(GRPOConfig):
    """Advantage = r - mean (no std), sequence-mean-token-scale aggregation."""
    algo_variant: str = "drgrpo"
    advantage_estimator: str = "drgrpo"
    loss_agg_mode: str = "sequence-mean-token-scale"


@dataclasses.dataclass(kw_only=True)
class PPOConfig(AlgorithmConfig):
    algo_variant: str = "ppo"
    advantage_estimator: str = "gae"
    policy_loss_fn: str = "ppo"
    value_loss_fn: str = "ppo"
    num_iterations: int = 1
    gamma: float = 1.0
    gae_lambda: float = 0.95
    beta: float = 0.04
    epsilon: float = 0.2
    epsilon_low: Optional[float] = None
    epsilon_high: Optional[float] = None
    epsilon_c: Optional[float] = None
    entropy_coef: Optional[float] = None
    clip_range_value: float = 0.2
    kl_method: str = "low_var_kl"
    loss_agg_mode: str = "token-mean"

    def __post_init__(self):
        super().__post_init__()
        if self.epsilon_low is None:
            self.epsilon_low = self.epsilon
        if self.epsilon_high is None:
            self.epsilon_high = self.epsilon
        if self.epsilon_c is not None and self.epsilon_c <= 1.0:
            raise ValueError("epsilon_c (dual-clip) must be > 1")
