"""Reward functions over graded math answers (tunix/utils/math_rewards.py:27-60)."""
from __future__ import annotations

from typing import List

from . import math_utils


def math_reward(prompts: List[str], completions: List[str], answer: List[str], **kwargs) -> List[float]:
    """1.0 when the completion's final answer (boxed / '####' / 'answer is') grades equal to `answer`, else 0.0."""
    out = []
    for completion, truth in zip(completions, answer):
        got = math_utils.extract_answer(completion)
        truth_val = math_utils.extract_answer(str(truth)) if ("\\boxed" in str(truth) or "####" in str(truth)) else str(truth)
        out.append(1.0 if got is not None and math_utils.grade_answer(got, truth_val) else 0.0)
    return out


def format_reward(prompts: List[str], completions: List[str], **kwargs) -> List[float]:
    """0.5 for completions that end in a boxed answer: a shaping term for early training."""
    return [0.5 if math_utils.extract_boxed_answer(c) is not None else 0.0 for c in completions]
