"""Reward managers (tunix/rl/reward_manager.py:73-430).

`sequence-level`: sums N reward functions per completion; algorithm-config attributes are injected into a
reward function when its signature names them (:289-305); optionally evaluated in a forkserver process pool
with a per-chunk timeout and per-function fallback to the parent process (:188-257). Returns the final
rewards plus the per-function columns for logging. `agentic-sequence-level` adds environment rewards
carried by trajectories (:380-430).
"""
from __future__ import annotations

import abc
import concurrent.futures as cf
import inspect
import multiprocessing as mp
import os
from typing import Any, Callable, Dict, List, Sequence

import numpy as np

from . import function_registry

RewardFn = Callable[..., Any]


class AbstractRewardManager(abc.ABC):
    def __init__(self, reward_fns, algo_config):
        self.reward_fns = [reward_fns] if not isinstance(reward_fns, Sequence) else list(reward_fns)
        if not self.reward_fns:
            raise ValueError("reward_fns cannot be empty. You must provide at least one reward function.")
        self.algo_config = algo_config

    @abc.abstractmethod
    def __call__(self, prompts: List[str], completions: List[str], **kwargs) -> Dict[str, Any]: ...


def _call_reward_fn(fn, prompts, completions, kwargs):
    return np.asarray(fn(prompts=prompts, completions=completions, **kwargs), dtype=np.float32)


@function_registry.register_reward_manager("sequence-level")
class SequenceRewardManager(AbstractRewardManager):
    def __init__(self, reward_fns, algo_config, **kwargs):
        super().__init__(reward_fns, algo_config)
        n = getattr(algo_config, "reward_num_workers", 0)
        self._num_workers = (os.cpu_count() or 1) if n == -1 else n
        self._timeout = getattr(algo_config, "reward_worker_timeout_seconds", 180.0)
        self._pool = None

    def _fn_kwargs(self, fn, kwargs: dict) -> dict:
        """Pass only what the function accepts; inject algo-config attributes named in its signature."""
        try:
            params = inspect.signature(fn).parameters
        except (TypeError, ValueError):
            return kwargs
        accepts_var = any(p.kind == inspect.Parameter.VAR_KEYWORD for p in params.values())
        out = dict(kwargs) if accepts_var else {k: v for k, v in kwargs.items() if k in params}
        for name in params:
            if name not in out and name not in ("prompts", "completions") and hasattr(self.algo_config, name):
                out[name] = getattr(self.algo_config, name)
        return out

    def _get_pool(self):
        if self._pool is None:
            self._pool = cf.ProcessPoolExecutor(self._num_workers, mp_context=mp.get_context("forkserver"))
        return self._pool

    def _run_fn(self, fn, prompts, completions, kwargs) -> np.ndarray:
        kw = self._fn_kwargs(fn, kwargs)
        if self._num_workers and self._num_workers > 0 and len(prompts) > 1:
            try:
                pool = self._get_pool()
                n = len(prompts)
                chunks = np.array_split(np.arange(n), min(self._num_workers, n))
                futs = []
                for idx in chunks:
                    sub_kw = {k: ([v[i] for i in idx] if isinstance(v, (list, tuple)) and len(v) == n else v)
                              for k, v in kw.items()}
                    futs.append(pool.submit(_call_reward_fn, fn, [prompts[i] for i in idx],
                                            [completions[i] for i in idx], sub_kw))
                parts = [f.result(timeout=self._timeout) for f in futs]
                return np.concatenate(parts)
            except Exception:
                pass  # unpicklable function, worker crash or timeout: evaluate in the parent
        return _call_reward_fn(fn, prompts, completions, kw)

    def __call__(self, prompts, completions, **kwargs) -> Dict[str, Any]:
        cols = {}
        total = np.zeros(len(prompts), np.float32)
        for fn in self.reward_fns:
            r = self._run_fn(fn, prompts, completions, kwargs)
            if r.shape != (len(prompts),):
                raise ValueError(f"reward function {getattr(fn, '__name__', fn)} returned shape {r.shape}, "
                                 f"expected ({len(prompts)},)")
            cols[getattr(fn, "__name__", type(fn).__name__)] = r
            total += np.nan_to_num(r, nan=0.0)
        return {"rewards": total, "per_fn": cols}

    def close(self):
        if self._pool is not None:
            self._pool.shutdown(wait=False, cancel_futures=True)
            self._pool = None


@function_registry.register_reward_manager("agentic-sequence-level")
class AgenticSequenceRewardManager(SequenceRewardManager):
    """Adds the environment's trajectory reward (kwarg `env_rewards`) to the function rewards."""

    def __call__(self, prompts, completions, **kwargs):
        env = kwargs.pop("env_rewards", None)
        out = super().__call__(prompts, completions, **kwargs) if self.reward_fns else \
            {"rewards": np.zeros(len(prompts), np.float32), "per_fn": {}}
        if env is not None:
            env = np.asarray(env, np.float32)
            out["rewards"] = out["rewards"] + env
            out["per_fn"]["env"] = env
        return out
