"""Dr. GRPO (tunix/rl/grpo/drgrpo_learner.py:28-39): advantages without the division by the group's standard deviation and
a constant length normalisation of the loss (both set by `DrGRPOConfig`)."""
from __future__ import annotations

from ..algorithm_config import DrGRPOConfig
from .grpo_learner import GRPOLearner


class DrGRPOLearner(GRPOLearner):
    def __init__(self, rl_cluster, reward_fns, algo_config: DrGRPOConfig, **kw):
        super().__init__(rl_cluster, reward_fns, algo_config, **kw)
