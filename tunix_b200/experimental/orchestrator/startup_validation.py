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
