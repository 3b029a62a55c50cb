"""Split-step trainer protocol of the distributed engine (tunix/experimental/train/abstract_trainer.py:30-226): the
orchestrator sends micro-batches one by one and decides when the optimizer steps."""
from __future__ import annotations

import abc
from typing import Any, Optional


class AbstractTrainer(abc.ABC):
    @abc.abstractmethod
    def fwd_bwd(self, batch: Any, is_last_microbatch: bool = False) -> dict:
        """Loss and gradients of one micro-batch; gradients accumulate until `update`."""

    @abc.abstractmethod
    def update(self) -> dict:
        """One optimizer step over everything accumulated since the last one."""

    @abc.abstractmethod
    def eval_step(self, batch: Any) -> dict: ...

    @abc.abstractmethod
    def fwd_only(self, batch: Any, fn=None) -> Any:
        """A forward pass without gradients (scoring)."""

    @abc.abstractmethod
    def save_checkpoint(self, step: Optional[int] = None, force: bool = False, custom_metadata: Optional[dict] = None) -> bool: ...

    @abc.abstractmethod
    def restore_checkpoint(self, step: Optional[int] = None) -> int: ...

    @property
    @abc.abstractmethod
    def train_steps(self) -> int: ...
