"""RL helpers (tunix/rl/utils.py): micro-batch slicing / merging, unpadding, streaming sequence packing
with an update-boundary flag (:521-657), pack-size arithmetic (:402-441), critic model builder (:253-319)."""
from __future__ import annotations

import dataclasses
from typing import Iterable, Iterator, Optional

import numpy as np
import torch
import torch.nn as nn

from . import common, packing


def chunk_slices(n: int, size: int) -> list[slice]:
    return [slice(i, min(i + size, n)) for i in range(0, n, max(size, 1))]


def slice_example(ex: common.TrainExample, sl: slice) -> common.TrainExample:
    kw = {}
    for f in dataclasses.fields(ex):
        v = getattr(ex, f.name)
        kw[f.name] = v[sl] if isinstance(v, torch.Tensor) and v.dim() >= 1 else v
    return common.TrainExample(**kw)


def merge_examples(examples: list[common.TrainExample]) -> common.TrainExample:
    kw = {}
    for f in dataclasses.fields(examples[0]):
        vals = [getattr(e, f.name) for e in examples]
        kw[f.name] = torch.cat(vals, 0) if isinstance(vals[0], torch.Tensor) and vals[0].dim() >= 1 else vals[0]
    return common.TrainExample(**kw)


def compute_pack_size(global_batch_tokens: int, budget: int) -> int:
    return max(1, -(-global_batch_tokens // budget))


def validate_packing_budget(budget: int, max_prompt_length: int, max_completion_length: int) -> None:
    if budget < max_prompt_length + max_completion_length:
        raise ValueError(f"packing budget {budget} is smaller than the longest possible sequence "
                         f"({max_prompt_length} + {max_completion_length})")


def unpad_train_example(ex: common.TrainExample, pad_id: int) -> list[packing.PackItem]:
    """Strip left padding of prompts and right padding of completions -> one PackItem per row."""
    items = []
    B = ex.prompt_ids.shape[0]
    pm = ex.prompt_mask.cpu().numpy() > 0
    cm = ex.completion_mask.cpu().numpy()
    pid, cid = ex.prompt_ids.cpu().numpy(), ex.completion_ids.cpu().numpy()
    adv = ex.advantages.cpu().numpy()
    for b in range(B):
        p = pid[b][pm[b]].astype(np.int32)
        valid = np.nonzero(cm[b] > 0)[0]
        c_len = int(valid[-1]) + 1 if len(valid) else 0
        c = cid[b][:c_len].astype(np.int32)
        a = adv[b][:c_len] if adv.ndim == 2 else np.full(c_len, adv[b], np.float32)
        per = {}
        for name in ("old_per_token_logps", "ref_per_token_logps", "sampler_is_weights"):
            v = getattr(ex, name)
            if v is not None:
                per[name] = v[b].float().cpu().numpy()[:c_len]
        items.append(packing.PackItem(prompt_ids=p, completion_ids=c, completion_mask=cm[b][:c_len].astype(np.float32),
                                      advantages=a.astype(np.float32), per_token=per))
    return items


def packed_chunk_to_examples(chunk: packing.PackedChunk, device, is_update_step: Optional[bool] = None,
                             num_segments: Optional[int] = None) -> common.TrainExample:
    """A packed chunk becomes a TrainExample whose `prompt_ids` is empty and whose completion side is the
    whole packed row (loss positions are selected by `completion_mask`)."""
    t = lambda a, dt=None: torch.from_numpy(np.ascontiguousarray(a)).to(device=device, dtype=dt) if a is not None else None  # noqa: E731
    n_bins, budget = chunk.ids.shape
    return common.TrainExample(
        prompt_ids=torch.zeros((n_bins, 0), dtype=torch.long, device=device),
        prompt_mask=torch.zeros((n_bins, 0), dtype=torch.int32, device=device),
        completion_ids=t(chunk.ids, torch.long), completion_mask=t(chunk.completion_mask),
        advantages=t(chunk.advantages), segment_ids=t(chunk.segment_ids, torch.int32),
        segment_positions=t(chunk.segment_positions, torch.int32),
        num_segments=num_segments or (int(max(chunk.num_real_segments or (0,))) + 1),
        old_per_token_logps=t(chunk.per_token.get("old_per_token_logps")),
        ref_per_token_logps=t(chunk.per_token.get("ref_per_token_logps")),
        sampler_is_weights=t(chunk.per_token.get("sampler_is_weights")), is_update_step=is_update_step)


def pack_sequences(examples: Iterable[common.TrainExample], budget: int, pack_size: int, pad_id: int, device,
                   max_segments: Optional[int] = None, pinned: bool = False) -> Iterator[common.TrainExample]:
    """Streaming FFD packing: buffers items until a chunk of `pack_size` rows fills, yields packed examples,
    flushes the remainder at the end. The last yielded example carries `is_update_step=True`."""
    buf: list = []
    pending: Optional[common.TrainExample] = None
    for ex in examples:
        buf.extend(unpad_train_example(ex, pad_id))
        chunks, left = packing.pack_core(buf, pack_size, budget, pad_id, max_segments, min_buffered_tokens=pack_size * budget,
                                         pinned=pinned)
        for ch in chunks:
            if pending is not None:
                yield pending
            pending = packed_chunk_to_examples(ch, device, is_update_step=False)
        buf = [buf[i] for i in left]
    if buf:
        chunks, left = packing.pack_core(buf, pack_size, budget, pad_id, max_segments, pinned=pinned)
        for ch in chunks:
            if pending is not None:
                yield pending
            pending = packed_chunk_to_examples(ch, device, is_update_step=False)
    if pending is not None:
        pending.is_update_step = True
        yield pending


class ScoreHead(nn.Module):
    """Decoder backbone + scalar head: critic (per-position value) or reward model."""

    def __init__(self, backbone, dtype=None):
        super().__init__()
        self.backbone = backbone
        D = backbone.config.embed_dim
        p = next(backbone.parameters())
        self.score = nn.Linear(D, 1, bias=False, device=p.device, dtype=dtype or p.dtype)
        nn.init.normal_(self.score.weight, std=1.0 / (D ** 0.5))
        self.config = backbone.config

    def forward(self, input_tokens, positions=None, cache=None, attention_mask=None, segment_ids=None, **kw):
        hidden, _ = self.backbone(input_tokens, positions=positions, attention_mask=attention_mask,
                                  segment_ids=segment_ids, skip_lm_head=True)
        return self.score(hidden).float()[..., 0]


def create_critic_model(actor_or_backbone, seed: int = 0) -> ScoreHead:
    """Critic initialised from a copy of the given decoder with a fresh scalar head."""
    import copy
    torch.manual_seed(seed)
    return ScoreHead(copy.deepcopy(actor_or_backbone))
