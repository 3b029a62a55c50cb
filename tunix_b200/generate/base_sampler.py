"""Sampler interface and output container (tunix/generate/base_sampler.py:30-111)."""
from __future__ import annotations

import abc
import dataclasses
from typing import Any, Optional

import numpy as np


@dataclasses.dataclass
class SamplerOutput:
    text: list
    logits: Optional[Any]
    tokens: Any                      # list[np.ndarray] (ragged) or np.ndarray (padded)
    padded_prompt_tokens: np.ndarray
    logprobs: Optional[list]
    routed_experts: Optional[list] = None
    prompt_lengths: Optional[np.ndarray] = None


class BaseSampler(abc.ABC):
    @property
    @abc.abstractmethod
    def transformer(self): ...

    @abc.abstractmethod
    def __call__(self, input_strings, max_generation_steps, max_prompt_length=None, temperature=0.0, top_p=None,
                 top_k=None, beam_size=None, seed=None, return_logits: bool = True, echo: bool = False,
                 pad_output: bool = False): ...

    @abc.abstractmethod
    def tokenize(self, input_string: str): ...

    def update_params(self, updated_weights: Any, filter_types=None) -> None:
        raise NotImplementedError(f"{type(self).__name__} does not implement update_params.")

    def delete_cache(self) -> None:
        pass

    def reinitialize_cache(self) -> None:
        pass
