"""Thread-safe name -> function registries (tunix/rl/function_registry.py:26-178)."""
from __future__ import annotations

import threading
from typing import Callable

_lock = threading.Lock()
_REG: dict = {"policy_loss_fn": {}, "value_loss_fn": {}, "advantage_estimator": {}, "reward_manager": {}}


def _register(kind: str, name: str):
    def deco(fn):
        with _lock:
            _REG[kind][name] = fn
        return fn
    return deco


def _get(kind: str, name: str) -> Callable:
    with _lock:
        if name not in _REG[kind]:
            raise ValueError(f"unknown {kind} {name!r}; registered: {sorted(_REG[kind])}")
        return _REG[kind][name]


def register_policy_loss_fn(name): return _register("policy_loss_fn", name)
def register_value_loss_fn(name): return _register("value_loss_fn", name)
def register_advantage_estimator(name): return _register("advantage_estimator", name)
def register_reward_manager(name): return _register("reward_manager", name)
def get_policy_loss_fn(name): return _get("policy_loss_fn", name)
def get_value_loss_fn(name): return _get("value_loss_fn", name)
def get_advantage_estimator(name): return _get("advantage_estimator", name)
def get_reward_manager(name): return _get("reward_manager", name)


def list_policy_loss_fns():
    with _lock:
        return sorted(_REG["policy_loss_fn"])


def list_value_loss_fns():
    with _lock:
        return sorted(_REG["value_loss_fn"])


def list_advantage_estimators():
    with _lock:
        return sorted(_REG["advantage_estimator"])


def list_reward_managers():
    with _lock:
        return sorted(_REG["reward_manager"])
