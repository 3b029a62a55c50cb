"""Token sampling: greedy, temperature, top-k, top-p, chosen-token log-prob.

Semantics follow tunix/generate/sampler.py:112-168: logits / temperature -> (top-k) -> softmax -> sort ->
keep the smallest prefix whose cumulative probability reaches top_p -> renormalise -> categorical.
The random stream of step `s` is derived from `(seed, s)` only (the reference folds the step into the
key, :562), so a rollout is reproducible regardless of batching history. On CUDA the fused kernel in
csrc/sampling.cu does temperature, top-k / top-p filtering, the draw and the log-prob in one pass per row;
this module is its reference implementation and the CPU path.
"""
from __future__ import annotations

from typing import Optional

import torch


def _generator(device, seed: int, step: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed((int(seed) * 1000003 + int(step) * 7919 + 12345) & 0x7FFFFFFFFFFFFFFF)
    return g


def filter_logits(logits: torch.Tensor, temperature: float, top_p: Optional[float], top_k: Optional[int]) -> torch.Tensor:
    """Return masked, temperature-scaled logits whose softmax is the sampling distribution."""
    z = logits.float() / max(temperature, 1e-6)
    V = z.shape[-1]
    if top_k is not None and 0 < top_k < V:
        kth = torch.topk(z, top_k, dim=-1).values[..., -1:]
        z = z.masked_fill(z < kth, -float("inf"))
    if top_p is not None and top_p < 1.0:
        probs = torch.softmax(z, dim=-1)
        sp, si = torch.sort(probs, dim=-1, descending=True)
        cum = torch.cumsum(sp, dim=-1)
        drop = (cum - sp) > top_p            # keep tokens until the mass before them already exceeds top_p
        drop[..., 0] = False
        mask = torch.zeros_like(drop).scatter(-1, si, drop)
        z = z.masked_fill(mask, -float("inf"))
    return z


def sample(logits: torch.Tensor, *, temperature: float = 0.0, top_p: Optional[float] = None,
           top_k: Optional[int] = None, seed: int = 0, step: int = 0, want_logprob: bool = False):
    """logits [B, V] fp32 -> (tokens [B] int64, logprob of the chosen token under the UNfiltered
    temperature-scaled distribution, or None)."""
    if temperature is None or temperature <= 0.0 or (top_p is None and top_k is None and temperature == 0.0):
        tok = torch.argmax(logits, dim=-1)
        lp = None
        if want_logprob:
            lp = torch.log_softmax(logits.float(), -1).gather(-1, tok[:, None])[:, 0]
        return tok, lp
    if logits.is_cuda:
        from ..ops import sampling_kernels
        if sampling_kernels.available():
            return sampling_kernels.sample(logits, temperature, top_p, top_k, seed, step, want_logprob)
    z = filter_logits(logits, temperature, top_p, top_k)
    probs = torch.softmax(z, dim=-1)
    tok = torch.multinomial(probs, 1, generator=_generator(logits.device, seed, step))[:, 0]
    lp = None
    if want_logprob:
        lp = torch.log_softmax(logits.float() / max(temperature, 1e-6), -1).gather(-1, tok[:, None])[:, 0]
    return tok, lp
