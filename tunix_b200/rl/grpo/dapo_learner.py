"""DAPO under its own module name (tunix/rl/grpo/dapo_learner.py:28-161); the implementation sits beside GRPO."""
from ..algorithm_config import DAPOConfig  # noqa: F401
from .grpo_learner import DAPOLearner  # noqa: F401

DapoConfig, DapoLearner = DAPOConfig, DAPOLearner
