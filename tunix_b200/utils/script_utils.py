"""Helpers shared by the example scripts (tunix/utils/script_utils.py:50-175): question / answer datasets for RL
recipes, and a context manager that captures a profile and the log of a code region."""
from __future__ import annotations

import logging
import os
from typing import Callable, Optional, Tuple

from ..examples.data import _records

DEBUG_LEVELS = {"DEBUG": logging.DEBUG, "INFO": logging.INFO, "WARNING": logging.WARNING, "ERROR": logging.ERROR,
                "FATAL": logging.CRITICAL}


class _Batches(list):
    """A list of batches with `repeat(n)` (the list n times over)."""

    def repeat(self, num_epochs: int) -> "_Batches":
        return _Batches(list(self) * int(num_epochs))


def get_dataset(path, split: str, seed: int, system_prompt: str, *, answer_extractor: Callable[[str], Optional[str]],
                dataset_name: str = "gsm8k") -> list:
    """Shuffled records `{"prompts", "question", "answer"}`: `prompts` (what the model sees) and `question` (what the
    reward functions see) are the system prompt followed by the question, `answer` is `answer_extractor(raw answer)`.
    `path` is a local file or directory (see `examples.data._records.load_records`); nothing is downloaded."""
    del dataset_name
    out = []
    for rec in _records.shuffled(_records.load_records(path, split), seed):
        q = system_prompt + str(rec["question"])
        out.append({"prompts": q, "question": q, "answer": answer_extractor(str(rec["answer"]))})
    return out


def get_train_and_eval_datasets(data_path, split: str, seed: int, system_prompt: str, batch_size: int, num_batches: Optional[int],
                                train_fraction: float, num_epochs: Optional[int], *,
                                answer_extractor: Callable[[str], Optional[str]], dataset_name: str = "gsm8k") -> Tuple[list, Optional[list]]:
    """(train batches, eval batches or None): records are batched (a short last batch is kept), cut to `num_batches`,
    split by `train_fraction`, and repeated `num_epochs` times; a batch is a dict of lists."""
    recs = get_dataset(data_path, split, seed, system_prompt, answer_extractor=answer_extractor, dataset_name=dataset_name)
    batches = _Batches({k: [r[k] for r in recs[i:i + batch_size]] for k in ("prompts", "question", "answer")}
                       for i in range(0, len(recs), batch_size))
    if num_batches:
        batches = _Batches(batches[:num_batches])
    if train_fraction == 1.0:
        return (batches.repeat(num_epochs) if num_epochs else batches), None
    n = int(len(batches) * train_fraction)
    train, val = _Batches(batches[:n]), _Batches(batches[n:])
    if num_epochs:
        train, val = train.repeat(num_epochs), val.repeat(num_epochs)
    return train, val


class profile_and_capture_log:
    """`with profile_and_capture_log("tag", log_dir=...):` records a `torch.profiler` trace of the region (CPU
    activity, CUDA activity when a GPU is present) under `<log_dir>/<tag>/` and copies the log records emitted inside
    the region to `<log_dir>/<tag>/captured.log`. Without `log_dir`, or with `enable_profile=False` and
    `capture_log=False`, it does nothing."""

    def __init__(self, tag: str = "", enable_profile: bool = True, log_dir: Optional[str] = None, capture_log: bool = True,
                 level: int = logging.INFO):
        self._dir = os.path.join(log_dir, tag or "profile") if log_dir else None
        self._profile, self._capture, self._level = enable_profile and log_dir is not None, capture_log and log_dir is not None, level
        self._prof = self._handler = None

    def __enter__(self):
        if self._dir is None:
            return self
        os.makedirs(self._dir, exist_ok=True)
        if self._capture:
            self._handler = logging.FileHandler(os.path.join(self._dir, "captured.log"))
            self._handler.setLevel(self._level)
            self._handler.setFormatter(logging.Formatter("%(asctime)s %(levelname)s %(name)s: %(message)s"))
            logging.getLogger().addHandler(self._handler)
        if self._profile:
            import torch
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self._prof = torch.profiler.profile(activities=acts)
            self._prof.start()
        return self

    def __exit__(self, *exc) -> bool:
        if self._prof is not None:
            self._prof.stop()
            self._prof.export_chrome_trace(os.path.join(self._dir, "trace.json"))
            self._prof = None
        if self._handler is not None:
            logging.getLogger().removeHandler(self._handler)
            self._handler.close()
            self._handler = None
        return False
