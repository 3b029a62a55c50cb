"""tqdm progress bar with a metrics postfix (tunix/sft/progress_bar.py:21-110)."""
from __future__ import annotations

from typing import Optional

try:
    from tqdm import tqdm
except Exception:  # pragma: no cover
    tqdm = None


class ProgressBar:
    def __init__(self, metrics_logger, initial_steps: int, max_steps: Optional[int], description: str = "Training",
                 metrics_prefix: str = "", disable: bool = False):
        self.metrics_logger = metrics_logger
        self.metrics_prefix = metrics_prefix
        self.metrics: dict = {}
        self.tqdm_bar = None
        if tqdm is not None and not disable:
            self.tqdm_bar = tqdm(total=max_steps, initial=initial_steps, desc=description, unit="step",
                                 dynamic_ncols=True, leave=True)

    def _update_metric(self, name: str, mode):
        if self.metrics_logger is None:
            return
        if self.metrics_logger.metric_exists(self.metrics_prefix, name, mode):
            self.metrics[f"{mode}_{name}"] = round(self.metrics_logger.get_metric(self.metrics_prefix, name, mode), 3)

    def update_metrics(self, names, mode, ndigits: int = 3):
        for n in names:
            self._update_metric(n, mode)
        if self.tqdm_bar is not None:
            self.tqdm_bar.set_postfix(self.metrics)

    def update(self, n: int = 1):
        if self.tqdm_bar is not None:
            self.tqdm_bar.update(n)

    def close(self):
        if self.tqdm_bar is not None:
            self.tqdm_bar.close()
