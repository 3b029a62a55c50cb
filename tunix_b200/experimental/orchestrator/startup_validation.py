"""Checks run before any worker does work (tunix/experimental/orchestrator/startup_validation.py:33-140): every
validator returns a list of messages, and one `StartupValidationError` carries all of them, so a misconfigured run
is told everything that is wrong at once instead of one error per attempt."""
from __future__ import annotations

from typing import Any, Optional, Protocol, Sequence


class StartupValidationError(ValueError):
    def __init__(self, errors: Sequence[str]):
        self.errors = list(errors)
        super().__init__("startup validation failed:\n" + "\n".join(f"  - {e}" for e in self.errors))


class StartupValidator(Protocol):
    def validate(self, registry, alg_config, training_config) -> list: ...


def _positive_int(value: Any, name: str, errors: list) -> bool:
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        errors.append(f"{name} must be a positive integer, got {value!r}")
        return False
    return True


class RunGeometryValidator:
    """Positive sizes, and the lattice mini batch -> micro batches / generation groups divides evenly."""

    def validate(self, registry, alg_config, training_config) -> list:
        errors: list = []
        g = getattr(alg_config, "num_generations", 1)
        mb = getattr(training_config, "mini_batch_size", None)
        _positive_int(getattr(alg_config, "max_response_length", 1024), "max_response_length", errors)
        g_ok = _positive_int(g, "num_generations", errors)
        mb_ok = _positive_int(mb, "mini_batch_size", errors)
        if g_ok and mb_ok and mb % g:
            errors.append(f"mini_batch_size {mb} is not divisible by num_generations {g}")
        packing = bool(getattr(training_config, "sequence_packing", False) or getattr(training_config, "pack_sequences", False))
        if mb_ok:
            for name in ("train_micro_batch_size", "rollout_micro_batch_size", "compute_logps_micro_batch_size"):
                v = getattr(training_config, name, None)
                if v is None or not _positive_int(v, name, errors):
                    continue
                if name == "train_micro_batch_size" and packing:
                    continue                                 # packed micro-batches are sized in tokens, not rows
                if mb % v:
                    errors.append(f"mini_batch_size {mb} is not divisible by {name} {v}")
        variant = getattr(alg_config, "algo_variant", "")
        if variant in ("grpo", "gspo-token") and g_ok and g <= 1:
            errors.append(f"num_generations must be > 1 for {variant!r}, got {g}")
        return errors


class RegistryValidator:
    """The roles a program needs are present, and (optionally) in the numbers the run was sized for."""

    def __init__(self, required_roles: Sequence[str] = ("trainer", "rollout"), min_counts: Optional[dict] = None):
        self.required_roles, self.min_counts = tuple(required_roles), dict(min_counts or {})

    def validate(self, registry, alg_config, training_config) -> list:
        errors = []
        for role in self.required_roles:
            n = len(registry.group(role))
            need = max(1, int(self.min_counts.get(role, 1)))
            if n < need:
                errors.append(f"role {role!r}: {n} worker(s) registered, {need} needed")
        return errors


DEFAULT_VALIDATORS = (RunGeometryValidator(), RegistryValidator())


def validate_startup(registry, alg_config, training_config, validators: Sequence[StartupValidator] = DEFAULT_VALIDATORS) -> None:
    errors: list = []
    for v in validators:
        errors += list(v.validate(registry, alg_config, training_config))
    if errors:
        raise StartupValidationError(errors)


def validate_program(program, engine) -> None:
    """The same all-at-once check for a `StandardRLProgram` on a `DistributedRLEngine`: the roles the program will call
    are served, the batch geometry can be assembled, and a window that lets rollouts run ahead comes with weight sync.
    `StandardRLProgram.run_async(..., validate=True)` calls it before the first dispatch."""
    errors: list = []
    rollout = getattr(engine, "_rollout", None)
    if rollout is not None and not rollout:
        errors.append("the engine has no rollout worker")
    trainers = getattr(engine, "_trainers", None)
    if trainers is not None and "actor" not in trainers:
        errors.append("the engine has no trainer worker for the actor role")
    if getattr(program, "reference_kl", False):
        serving = set(getattr(engine, "_inference", {}) or {}) | set(trainers or {})
        if "reference" not in serving:
            errors.append("reference_kl is on, but no worker serves the reference role")
    _positive_int(getattr(program, "num_generations", None), "num_generations", errors)
    _positive_int(getattr(program, "full_batch_size", None), "batch_size", errors)
    cfg = getattr(getattr(program, "assembler", None), "cfg", None)
    if cfg is not None:
        _positive_int(cfg.rows_per_microbatch, "rows_per_microbatch", errors)
        limit = getattr(program, "max_response_length", None) or getattr(getattr(program, "generation_args", None), "max_tokens", None)
        packed = type(program.assembler).__name__.startswith("SequencePacked")
        if packed and limit and limit + 1 > cfg.max_packed_len:
            errors.append(f"a response of up to {limit} tokens cannot fit a packed row of {cfg.max_packed_len} tokens")
        if not packed and limit and limit > cfg.max_response_length:
            errors.append(f"responses of up to {limit} tokens are cut to the assembler's max_response_length {cfg.max_response_length}")
    if getattr(program, "max_staleness", 0) > 0 and not getattr(program, "sync_weights", True):
        errors.append("max_staleness > 0 lets rollouts run ahead of the trainer, but sync_weights is off: the workers would never "
                      "see new weights")
    if getattr(program, "dataset", None) is None:
        errors.append("the program has no dataset")
    if errors:
        raise StartupValidationError(errors)
