"""Trainer-side helpers: deferred-division metrics, masks, positions, HBM report.

WeightedMetric / LossOutput follow tunix/sft/utils.py:186-306: a loss is carried as
(unreduced sum, denominator) so micro-batches of unequal token counts combine exactly.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Optional

import torch


@dataclasses.dataclass
class WeightedMetric:
    sum: torch.Tensor
    denominator: torch.Tensor
    eps: float = 0.0
    min_denominator: float = 0.0

    def value(self) -> torch.Tensor:
        d = self.denominator + self.eps
        if self.min_denominator:
            d = torch.clamp(d, min=self.min_denominator)
        return self.sum / d


@dataclasses.dataclass
class LossOutput:
    loss: WeightedMetric
    aux: Optional[dict] = None


def weighted_metric_mean(metrics: list[WeightedMetric]):
    """Global mean over micro-batches: sum of numerators over sum of denominators."""
    num = sum(float(m.sum) for m in metrics)
    den = sum(float(m.denominator) for m in metrics)
    eps = metrics[0].eps if metrics else 0.0
    mind = metrics[0].min_denominator if metrics else 0.0
    den = den + eps
    if mind:
        den = max(den, mind)
    return num / den if den != 0 else 0.0


def make_causal_attn_mask(input_mask: torch.Tensor) -> torch.Tensor:
    """[B,T] validity -> [B,T,T] boolean causal mask (tunix/sft/utils.py:35-56)."""
    B, T = input_mask.shape
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool, device=input_mask.device))
    return causal[None] & input_mask.bool()[:, None, :]


def build_positions_from_mask(input_mask: torch.Tensor) -> torch.Tensor:
    """Positions that count only valid tokens (left padding gets position 0) (tunix/sft/utils.py:59-72)."""
    m = input_mask.to(torch.int32)
    pos = torch.cumsum(m, dim=-1) - 1
    return torch.clamp(pos, min=0).to(torch.int32)


def is_lora_enabled(model) -> bool:
    from ..lora import is_lora_enabled as _f
    return _f(model)


def show_hbm_usage(title: str = "") -> dict:
    """Per-device memory in use / peak (tunix/sft/utils.py:153-183)."""
    out = {}
    if torch.cuda.is_available():
        for d in range(torch.cuda.device_count()):
            st = torch.cuda.memory_stats(d)
            out[d] = {"in_use": st.get("allocated_bytes.all.current", 0), "peak": st.get("allocated_bytes.all.peak", 0),
                      "limit": torch.cuda.get_device_properties(d).total_memory}
    if title:
        fmt = ", ".join(f"cuda:{d} {v['in_use'] / 2**30:.2f}/{v['limit'] / 2**30:.0f} GiB" for d, v in out.items())
        print(f"[hbm] {title}: {fmt or 'no CUDA device'}")
    return out


def try_get_learning_rate(optimizer: Any, step: int) -> Optional[float]:
    fn = getattr(optimizer, "learning_rate_at", None)
    if fn is None:
        return None
    try:
        return float(fn(step))
    except Exception:  # pragma: no cover
        return None
