"""DAPO (tunix/rl/grpo/dapo_learner.py:28-161): GRPO without the KL term, with clip-higher, token-mean aggregation
and the overlong-buffer reward shaping."""
from __future__ import annotations

import numpy as np

from ..algorithm_config import DAPOConfig
from .grpo_learner import GRPOLearner

DapoConfig = DAPOConfig


class DAPOLearner(GRPOLearner):
    """beta = 0, clip-higher, token-mean aggregation, overlong-buffer reward shaping (soft length penalty)."""

    def __init__(self, rl_cluster, reward_fns, algo_config: DAPOConfig, **kw):
        super().__init__(rl_cluster, reward_fns, algo_config, **kw)

    def _shape_rewards(self, rewards, completions, lengths):
        ob = getattr(self.algo_config, "overlong_buffer", None)
        if not ob or not ob.get("enable", False):
            return rewards
        buf = ob["overlong_buffer_length"]
        penalty = ob.get("overlong_buffer_penalty", 1.0)
        max_len = ob["max_response_length"]
        expected = max_len - buf
        # the reference measures completion length in characters (tunix/rl/grpo/dapo_learner.py:127-133);
        # token counts are what the budget is about, so tokens are used here.
        exceed = np.asarray(lengths, np.float32) - expected
        shaped = np.minimum(-exceed / max(buf, 1) * penalty, 0.0)
        return rewards + shaped.astype(np.float32)


DapoLearner = DAPOLearner
