"""Training / data hooks (tunix/sft/hooks.py:25-77)."""
from __future__ import annotations

import abc
from typing import Any, Optional


class TrainingHooks(abc.ABC):
    def on_train_start(self, train_ctx) -> None: ...
    def on_train_end(self, train_ctx) -> None: ...
    def on_train_step_start(self, train_ctx) -> None: ...
    def on_train_step_end(self, train_ctx, train_step: int, train_loss: float) -> None: ...
    def on_eval_step_start(self, train_ctx) -> None: ...
    def on_eval_step_end(self, train_ctx, eval_loss: float) -> None: ...


class DataHooks(abc.ABC):
    """External batch loaders: return the next batch or None at the end of the data."""

    def load_next_train_batch(self, train_ctx) -> Optional[Any]:
        return None

    def load_next_eval_batch(self, train_ctx) -> Optional[Any]:
        return None
