"""Hyper-parameter loading for the command-line entry points (tunix/cli/config.py:381-1220).

Precedence: base YAML (first positional argument) <- `override_config_file=<yaml>` <- `key=value` arguments
with dotted paths (`training_config.max_steps=20`) and `T_`-prefixed environment variables (`T_BATCH_SIZE=8`).
Giving the same key on the command line and in the environment is an error (:968-975). Values are parsed as
YAML scalars and type-checked against the base file (:1012-1045); sections listed in `replace_keys` are
replaced wholesale instead of merged (:431-437); per-role model configs inherit from `model_config`
(:456-470). The optimizer factory builds `tunix_b200.optim` optimizers with schedule kwargs filtered by
signature (:210-378); reward functions are loaded from file or dotted paths (:1124-1220).
"""
from __future__ import annotations

import copy
import importlib
import importlib.util
import inspect
import os
import re
import sys
from typing import Any, Callable, Optional

import yaml

from .. import optim as optim_lib

REPLACE_KEYS = ("lora_config", "reward_functions", "config_overrides", "vllm_config", "sglang_jax_config")
ROLE_MODEL_KEYS = ("actor_model_config", "critic_model_config", "reference_model_config", "rollout_model_config",
                   "reward_model_config")


def _unalias(obj: Any) -> Any:
    """A copy in which no two places share a container (`<<: *anchor` merges reuse the anchor's nested objects)."""
    if isinstance(obj, dict):
        return {k: _unalias(v) for k, v in obj.items()}
    if isinstance(obj, list):
        return [_unalias(v) for v in obj]
    return obj


_SCI_NUMBER = re.compile(r"^[+-]?(\d+\.?\d*|\.\d+)[eE][+-]?\d+$")


def _fix_numbers(obj: Any) -> Any:
    """YAML 1.1 reads `3e-4` (no dot in the mantissa) as a string; here it is the number it looks like, in override
    values and in override files alike."""
    if isinstance(obj, str) and _SCI_NUMBER.match(obj.strip()):
        return float(obj)
    if isinstance(obj, dict):
        return {k: _fix_numbers(v) for k, v in obj.items()}
    if isinstance(obj, list):
        return [_fix_numbers(v) for v in obj]
    return obj


def _parse_scalar(text: str) -> Any:
    try:
        return _fix_numbers(yaml.safe_load(text))
    except yaml.YAMLError:
        return text


def _set_path(cfg: dict, dotted: str, value: Any, schema: Optional[dict], strict_types: bool = True) -> None:
    parts = dotted.split(".")
    node, snode = cfg, schema
    for p in parts[:-1]:
        if not isinstance(node.get(p), dict):
            node[p] = {}
        node = node[p]
        snode = snode.get(p) if isinstance(snode, dict) else None
    leaf = parts[-1]
    if isinstance(snode, dict) and leaf in snode and snode[leaf] is not None and strict_types:
        want = snode[leaf]
        ok = isinstance(value, type(want)) or (isinstance(want, float) and isinstance(value, int)) or value is None \
            or (isinstance(want, bool) and isinstance(value, bool))
        if isinstance(want, bool) != isinstance(value, bool) and value is not None:
            ok = False
        if not ok:
            raise TypeError(f"override {dotted}={value!r} has type {type(value).__name__}, base config has "
                            f"{type(want).__name__}")
    node[leaf] = value


def _merge(base: dict, over: dict, path: str = "") -> dict:
    out = copy.deepcopy(base)
    for k, v in over.items():
        if isinstance(v, dict) and isinstance(out.get(k), dict) and k not in REPLACE_KEYS:
            out[k] = _merge(out[k], v, f"{path}{k}.")
        else:
            out[k] = copy.deepcopy(v)
    return out


class HyperParameters:
    def __init__(self, argv: list[str], env: Optional[dict] = None):
        """argv[0] is the program name, argv[1] the base YAML; the rest are key=value overrides."""
        if len(argv) < 2:
            raise ValueError("usage: <main> base_config.yaml [override_config_file=path] [key=value ...]")
        env = os.environ if env is None else env
        base_path = argv[1]
        if not os.path.exists(base_path):
            cand = os.path.join(os.path.dirname(os.path.abspath(__file__)), base_path)
            base_path = cand if os.path.exists(cand) else base_path
        with open(base_path) as f:
            base = _unalias(_fix_numbers(yaml.safe_load(f)))       # YAML anchors make sections share nested dicts: give each its own
        self._schema = copy.deepcopy(base)
        cfg = base
        cli: dict = {}
        for arg in argv[2:]:
            if "=" not in arg:
                raise ValueError(f"override {arg!r} is not of the form key=value")
            k, v = arg.split("=", 1)
            cli[k.strip()] = v
        if "override_config_file" in cli:
            with open(cli.pop("override_config_file")) as f:
                cfg = _merge(cfg, _fix_numbers(yaml.safe_load(f) or {}))
        env_over = {}
        for k, v in env.items():
            if k.startswith("T_"):
                key = k[2:].lower()
                if key in self._schema:
                    env_over[key] = v
        both = set(cli) & set(env_over)
        if both:
            raise ValueError(f"keys given both on the command line and in the environment: {sorted(both)}")
        for k, v in {**env_over, **cli}.items():
            top = k.split(".")[0]
            if top not in self._schema:
                raise KeyError(f"unknown config key {k!r}")
            _set_path(cfg, k, _parse_scalar(v), self._schema)
        # role model configs inherit from model_config
        for role in ROLE_MODEL_KEYS:
            if cfg.get(role) is not None:
                cfg[role] = _merge(cfg["model_config"], {k: v for k, v in cfg[role].items()
                                                         if v != self._schema["model_config"].get(k)})
        self.config = cfg
        self._validate()

    def _validate(self) -> None:
        c = self.config
        if c["batch_size"] <= 0:
            raise ValueError("batch_size must be positive")
        if c["rollout_engine"] not in ("vanilla", "paged"):
            raise ValueError(f"rollout_engine must be 'vanilla' or 'paged', got {c['rollout_engine']!r}")
        m = c["model_config"]["mesh"]
        from ..parallel.mesh import create_mesh  # noqa: F401  (parsing check only)
        import ast
        shape, names = ast.literal_eval(m["shape"]), ast.literal_eval(m["axis_names"])
        if len(shape) != len(names):
            raise ValueError(f"mesh shape {shape} and axis names {names} differ in length")

    def __getitem__(self, key: str) -> Any:
        return self.config[key]

    def get(self, key: str, default=None) -> Any:
        return self.config.get(key, default)

    # ---------------------------------------------------------------- factories
    def create_optimizer(self, section: str = "optimizer_config", parent: Optional[str] = None, max_steps: Optional[int] = None):
        oc = (self.config[parent][section] if parent else self.config[section]) or {}
        return create_optimizer(oc, max_steps or self.config["training_config"].get("max_steps"))

    def create_mesh(self, section: str = "model_config"):
        from ..parallel.mesh import create_mesh
        m = self.config[section]["mesh"]
        import ast

        import numpy as np
        import torch.distributed as dist
        if not dist.is_initialized():
            return None
        shape = ast.literal_eval(m["shape"]) if isinstance(m["shape"], str) else m["shape"]
        shape = (shape,) if isinstance(shape, int) else tuple(shape)
        world = dist.get_world_size()
        if int(np.prod(shape)) == 1 and world > 1 and len(shape) == 1:
            shape = (world,)          # the default "(1,)" means "all ranks along the one axis"
        if int(np.prod(shape)) != world:
            raise ValueError(f"{section}.mesh.shape {shape} needs {int(np.prod(shape))} ranks, the job has {world}")
        return create_mesh(shape, m["axis_names"])

    def obtain_reward_fns(self) -> list[Callable]:
        return [load_reward_fn(p) for p in (self.config.get("reward_functions") or [])]


def create_optimizer(oc: dict, max_steps: Optional[int] = None) -> optim_lib.Optimizer:
    oc = dict(oc)
    sched = oc.get("schedule_type")
    sk = dict(oc)
    if sched and "warmup_ratio" in oc and max_steps and not oc.get("warmup_steps"):
        sk["warmup_steps"] = int(oc["warmup_ratio"] * max_steps)
    if sched and max_steps and not oc.get("decay_steps"):
        sk["decay_steps"] = max_steps
    return optim_lib.create_optimizer(
        oc.get("opt_type", "adamw"), learning_rate=oc.get("learning_rate"), schedule_type=sched, schedule_kwargs=sk,
        max_grad_norm=oc.get("max_grad_norm"), **{k: oc[k] for k in ("b1", "b2", "eps", "weight_decay", "momentum") if k in oc})


def load_reward_fn(path: str) -> Callable:
    """`pkg.module:fn`, `pkg.module.fn` or `path/to/file.py[:fn]` (default: the first public function named `*reward*`)."""
    fn_name = None
    if path.endswith(".py") or ".py:" in path:
        if ":" in path:
            path, fn_name = path.rsplit(":", 1)
        if not os.path.isabs(path) and not os.path.exists(path):
            root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
            path = os.path.join(root, path)
        spec = importlib.util.spec_from_file_location(os.path.splitext(os.path.basename(path))[0], path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    else:
        if ":" in path:
            mod_name, fn_name = path.split(":", 1)
        else:
            mod_name, fn_name = path.rsplit(".", 1)
        mod = importlib.import_module(mod_name)
    if fn_name:
        return getattr(mod, fn_name)
    cands = [f for n, f in inspect.getmembers(mod, inspect.isfunction) if "reward" in n and not n.startswith("_")
             and f.__module__ == mod.__name__]
    if not cands:
        raise ValueError(f"no reward function found in {path}")
    return cands[0]
