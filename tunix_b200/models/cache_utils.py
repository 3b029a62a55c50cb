"""KV-cache bookkeeping shared by samplers (tunix/models/cache_utils.py:1-419): prefix-length bucketing, ring-buffer
(sliding-window) write positions, chunked-prefill slices and the masks that go with them.

Everything here is index arithmetic on small host or device tensors; the data movement itself is done by the
attention / paged-KV kernels."""
from __future__ import annotations

from typing import Optional, Sequence

import torch


def prefix_bucket_boundaries(max_length: int, step: int = 512) -> list:
    """Linear buckets `step, 2*step, ...` up to max_length: every bucket is one captured graph / one shape."""
    out = list(range(step, max_length + 1, step))
    if not out or out[-1] < max_length:
        out.append(max_length)
    return out


def bucket_prefix_length(length: int, boundaries: Sequence[int]) -> int:
    for b in boundaries:
        if length <= b:
            return b
    raise ValueError(f"prefix of {length} tokens exceeds the largest bucket {boundaries[-1]}")


def ring_positions(start: int, count: int, cache_len: int, device=None) -> torch.Tensor:
    """Slots written by tokens at absolute positions [start, start + count) in a ring buffer of `cache_len`."""
    return (torch.arange(start, start + count, device=device) % cache_len).to(torch.int64)


def ring_slot_positions(end_index: int, cache_len: int, device=None) -> torch.Tensor:
    """Absolute position held by each slot after `end_index` tokens were written (-1 = never written)."""
    slots = torch.arange(cache_len, device=device)
    if end_index <= cache_len:
        return torch.where(slots < end_index, slots, torch.full_like(slots, -1))
    wraps = (end_index - 1 - slots) // cache_len
    return slots + wraps * cache_len


def decode_mask(slot_pos: torch.Tensor, query_pos: int, window: Optional[int] = None) -> torch.Tensor:
    """[cache_len] bool: slots a query at `query_pos` may attend to (causal, optionally the last `window` tokens)."""
    ok = (slot_pos >= 0) & (slot_pos <= query_pos)
    if window:
        ok &= slot_pos > query_pos - window
    return ok


def prefill_mask(q_pos: torch.Tensor, k_pos: torch.Tensor, window: Optional[int] = None,
                 bidirectional_span: Optional[torch.Tensor] = None) -> torch.Tensor:
    """[Tq, Tk] bool causal (band-limited when `window`) mask; tokens sharing a positive id in
    `bidirectional_span` (image tokens of one image) also see each other both ways."""
    m = k_pos[None, :] <= q_pos[:, None]
    if window:
        m &= k_pos[None, :] > q_pos[:, None] - window
    if bidirectional_span is not None:
        s = bidirectional_span
        m |= (s[:, None] == s[None, :]) & (s[:, None] > 0)
    return m & (k_pos[None, :] >= 0)


def chunked_prefill_slices(prompt_len: int, chunk: int) -> list:
    """(start, stop) token ranges of a prompt prefilled `chunk` tokens at a time."""
    return [(s, min(s + chunk, prompt_len)) for s in range(0, prompt_len, chunk)]


def shared_kv_source_layers(layer_types: Sequence[str], frac_shared: float) -> list:
    """KV-cache sharing pattern of Gemma-4 style models: the last `frac_shared` of the layers do not keep their
    own cache but read the cache of the last unshared layer of the same attention type. Returns, per layer, the
    index of the layer whose cache it uses (itself when unshared)."""
    L = len(layer_types)
    first_shared = L - int(round(L * frac_shared))
    last_of_type = {}
    out = []
    for i, t in enumerate(layer_types):
        if i < first_shared:
            last_of_type[t] = i
            out.append(i)
        else:
            if t not in last_of_type:
                raise ValueError(f"layer {i} ({t}) has no unshared layer of its type to borrow a cache from")
            out.append(last_of_type[t])
    return out
