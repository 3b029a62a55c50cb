"""Pool feature maps of different widths to a common shape (tunix/distillation/feature_extraction/pooling.py)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def avg_pool_to(x: torch.Tensor, target_dim: int) -> torch.Tensor:
    """[..., D] -> [..., target_dim] by adaptive average pooling over the feature dim."""
    if x.shape[-1] == target_dim:
        return x
    lead = x.shape[:-1]
    return F.adaptive_avg_pool1d(x.reshape(-1, 1, x.shape[-1]).float(), target_dim).reshape(*lead, target_dim)


def pool_sequence(x: torch.Tensor, mask: torch.Tensor | None = None) -> torch.Tensor:
    """[B, T, D] -> [B, D] masked mean over time."""
    if mask is None:
        return x.float().mean(1)
    m = mask.float().unsqueeze(-1)
    return (x.float() * m).sum(1) / m.sum(1).clamp(min=1.0)
