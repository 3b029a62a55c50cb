"""Dr. GRPO under its own module name (tunix/rl/grpo/drgrpo_learner.py:28-39); the implementation sits beside GRPO."""
from ..algorithm_config import DrGRPOConfig  # noqa: F401
from .grpo_learner import DrGRPOLearner  # noqa: F401
