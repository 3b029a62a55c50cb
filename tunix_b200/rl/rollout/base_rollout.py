"""Rollout worker interface (tunix/rl/rollout/base_rollout.py:34-112)."""
from __future__ import annotations

import abc
import dataclasses
from typing import Any, Optional

import numpy as np


@dataclasses.dataclass
class RolloutOutput:
    text: list
    logits: Optional[list]
    tokens: list                       # list[np.ndarray], ragged completions
    left_padded_prompt_tokens: np.ndarray
    logprobs: Optional[list]
    routed_experts: Optional[list] = None
    prompt_lengths: Optional[np.ndarray] = None


class BaseRollout(abc.ABC):
    @abc.abstractmethod
    def generate(self, prompts, rollout_config, **kwargs) -> RolloutOutput: ...

    @abc.abstractmethod
    def get_per_token_logps(self, prompt_tokens, completion_tokens, completion_mask=None): ...

    @abc.abstractmethod
    def update_params(self, params, filter_types=None) -> None: ...

    @abc.abstractmethod
    def pad_id(self) -> int: ...

    @abc.abstractmethod
    def eos_id(self) -> int: ...

    @abc.abstractmethod
    def model(self) -> Any: ...
