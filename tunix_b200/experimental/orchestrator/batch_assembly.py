"""Batch assembly between rollout and trainer (tunix/experimental/orchestrator/batch_assembly.py:44-1413).

Unbatched `RLTrainerPayload`s (one trajectory each) are fed as they arrive; micro-batches come out when enough
have accumulated, the tail with `flush()`:

  `PaddedBatchAssembler`           rectangular `[rows, max_prompt + max_response]`: prompts left-padded,
                                   completions right-padded, one trajectory per row
  `SequencePackedBatchAssembler`   several trajectories per row of `max_packed_len` tokens (first-fit-decreasing
                                   through the native packing extension, `rl.packing`), with segment ids and
                                   per-segment positions for the flash-attention kernels

Every batch carries `PaddingStats` (how full the rows are) and a `LineageContext` whose parents are the
trajectories it was made from."""
from __future__ import annotations

import dataclasses
from typing import Any, Iterator, NamedTuple, Optional, Sequence

import numpy as np

from ...rl import packing
from ..common.datatypes import RLTrainerPayload
from ..common.lineage import LineageContext


@dataclasses.dataclass(frozen=True, kw_only=True)
class PaddingStats:
    row_valid_tokens: np.ndarray     # [rows] real tokens per row
    row_num_sequences: np.ndarray    # [rows] trajectories per row (0 = filler row)
    row_capacity: int

    def __post_init__(self):
        if self.row_valid_tokens.ndim != 1 or self.row_valid_tokens.size == 0:
            raise ValueError("row_valid_tokens must be a non-empty 1-D array")
        if self.row_num_sequences.shape != self.row_valid_tokens.shape:
            raise ValueError("row_num_sequences must match row_valid_tokens")
        if self.row_capacity <= 0:
            raise ValueError(f"row_capacity must be positive, got {self.row_capacity}")
        if (self.row_valid_tokens < 0).any() or (self.row_valid_tokens > self.row_capacity).any():
            raise ValueError("row_valid_tokens must lie in [0, row_capacity]")

    @property
    def num_rows(self) -> int:
        return int(self.row_valid_tokens.size)

    @property
    def valid_tokens(self) -> int:
        return int(self.row_valid_tokens.sum())

    @property
    def capacity_tokens(self) -> int:
        return self.num_rows * self.row_capacity

    @property
    def padding_ratio(self) -> float:
        return 1.0 - self.valid_tokens / self.capacity_tokens

    @property
    def row_fill(self) -> np.ndarray:
        return self.row_valid_tokens / float(self.row_capacity)

    @property
    def row_imbalance(self) -> float:
        """Fullest row over the mean row (1.0 = perfectly even); what the slowest data-parallel rank sees."""
        mean = self.row_valid_tokens.mean()
        return float(self.row_valid_tokens.max() / mean) if mean > 0 else 1.0


class AssembledBatch(NamedTuple):
    batch_id: str
    arrays: dict                 # name -> np.ndarray, what the trainer's input function takes
    stats: PaddingStats
    lineage: LineageContext
    num_trajectories: int


@dataclasses.dataclass(frozen=True, kw_only=True)
class BatchConfig:
    rows_per_microbatch: int = 8
    max_prompt_length: int = 256
    max_response_length: int = 768
    max_packed_len: int = 4096
    max_segments_per_row: Optional[int] = None
    pad_id: int = 0
    rollouts_per_optimizer_update: int = 64


def _example_fields(item: RLTrainerPayload):
    ex = item.example
    get = (lambda k, d=None: ex.get(k, d)) if isinstance(ex, dict) else (lambda k, d=None: getattr(ex, k, d))
    prompt = np.asarray(get("prompt_ids"), np.int32).reshape(-1)
    comp = np.asarray(get("completion_ids"), np.int32).reshape(-1)
    mask = get("completion_mask")
    mask = np.ones(len(comp), np.float32) if mask is None else np.asarray(mask, np.float32).reshape(-1)
    adv = get("advantages")
    if adv is None:
        adv = np.full(len(comp), 0.0 if item.reward is None else item.reward, np.float32)
    adv = np.broadcast_to(np.asarray(adv, np.float32).reshape(-1), comp.shape).copy()
    per_token = {k: np.asarray(get(k), np.float32).reshape(-1) for k in packing.PER_TOKEN_FIELDS if get(k) is not None}
    return prompt, comp, mask, adv, per_token


def _lineage_of(item) -> Optional[LineageContext]:
    ex = item.example
    lin = ex.get("lineage") if isinstance(ex, dict) else getattr(ex, "lineage", None)
    return lin if isinstance(lin, LineageContext) else None


class _Base:
    def __init__(self, cfg: BatchConfig, start_batch_index: int = 0):
        self.cfg = cfg
        self._buf: list = []
        self._next = start_batch_index

    @property
    def rollouts_per_optimizer_update(self) -> int:
        return self.cfg.rollouts_per_optimizer_update

    def reset(self, *, start_batch_index: Optional[int] = None) -> None:
        self._buf = []
        if start_batch_index is not None:
            self._next = start_batch_index

    def feed(self, items: Sequence[RLTrainerPayload]) -> Iterator[AssembledBatch]:
        self._buf.extend(items)
        yield from self._drain(drain_all=False)

    def flush(self) -> Iterator[AssembledBatch]:
        yield from self._drain(drain_all=True)

    def _batch_id(self) -> str:
        bid = f"batch_{self._next}"
        self._next += 1
        return bid

    def _lineage(self, bid: str, items, op: str, attrs: dict) -> LineageContext:
        return LineageContext.merge(bid, [_lineage_of(i) for i in items], "orchestrator.assembler", op, attrs)


class PaddedBatchAssembler(_Base):
    def _drain(self, drain_all: bool):
        R = self.cfg.rows_per_microbatch
        while len(self._buf) >= R or (drain_all and self._buf):
            items, self._buf = self._buf[:R], self._buf[R:]
            yield self._emit(items)

    def _emit(self, items) -> AssembledBatch:
        cfg = self.cfg
        R, P, C = cfg.rows_per_microbatch, cfg.max_prompt_length, cfg.max_response_length
        ids = np.full((R, P + C), cfg.pad_id, np.int32)
        pmask = np.zeros((R, P + C), np.float32)
        cmask = np.zeros((R, P + C), np.float32)
        adv = np.zeros((R, P + C), np.float32)
        extra: dict = {}
        valid = np.zeros(R, np.int64)
        for r, it in enumerate(items):
            prompt, comp, mask, a, per_token = _example_fields(it)
            prompt, comp, mask, a = prompt[-P:], comp[:C], mask[:C], a[:C]
            ids[r, P - len(prompt):P] = prompt
            pmask[r, P - len(prompt):P] = 1
            ids[r, P:P + len(comp)] = comp
            cmask[r, P:P + len(comp)] = mask
            adv[r, P:P + len(comp)] = a
            for k, v in per_token.items():
                extra.setdefault(k, np.zeros((R, P + C), np.float32))[r, P:P + len(comp)] = v[:C]
            valid[r] = len(prompt) + len(comp)
        bid = self._batch_id()
        stats = PaddingStats(row_valid_tokens=valid, row_num_sequences=(valid > 0).astype(np.int64), row_capacity=P + C)
        arrays = {"input_tokens": ids, "prompt_mask": pmask, "completion_mask": cmask, "advantages": adv, **extra}
        return AssembledBatch(bid, arrays, stats, self._lineage(bid, items, "pad", {"rows": R, "padding_ratio": stats.padding_ratio}),
                              len(items))


class SequencePackedBatchAssembler(_Base):
    def _drain(self, drain_all: bool):
        cfg = self.cfg
        while self._buf:
            tokens = sum(len(_example_fields(i)[0]) + len(_example_fields(i)[1]) for i in self._buf)
            if not drain_all and tokens < cfg.rows_per_microbatch * cfg.max_packed_len:
                return                    # not enough to fill a micro-batch yet
            pack_items = []
            for it in self._buf:
                prompt, comp, mask, adv, per_token = _example_fields(it)
                pack_items.append(packing.PackItem(prompt_ids=prompt, completion_ids=comp, completion_mask=mask, advantages=adv,
                                                   per_token=per_token,
                                                   policy_version=np.asarray([it.policy_version], np.int32)))
            max_seg = cfg.max_segments_per_row or cfg.max_packed_len
            bins, starts, leftover = packing.fill_one_chunk(pack_items, cfg.rows_per_microbatch, cfg.max_packed_len, max_seg)
            if len(leftover) == len(pack_items):
                raise ValueError("a trajectory is longer than max_packed_len and can never be placed")
            bins = [b for b in bins if b]
            chunk = packing.pack_chunk(pack_items, bins, starts, cfg.max_packed_len, cfg.pad_id)
            used = [i for b in bins for i in b]
            items = [self._buf[i] for i in used]
            self._buf = [self._buf[i] for i in leftover]
            R = cfg.rows_per_microbatch
            arrays = {"input_tokens": chunk.ids, "prompt_mask": chunk.prompt_mask, "completion_mask": chunk.completion_mask,
                      "advantages": chunk.advantages, "segment_ids": chunk.segment_ids, "positions": chunk.segment_positions,
                      **dict(chunk.per_token)}
            rows = chunk.ids.shape[0]
            if rows < R:                                   # keep the micro-batch shape static: all-padding filler rows
                arrays = {k: np.concatenate([v, np.full((R - rows,) + v.shape[1:], cfg.pad_id if k == "input_tokens" else 0, v.dtype)])
                          for k, v in arrays.items()}
            valid = (arrays["segment_ids"] > 0).sum(-1).astype(np.int64)
            nseq = np.asarray(list(chunk.num_real_segments) + [0] * (R - rows), np.int64)
            stats = PaddingStats(row_valid_tokens=valid, row_num_sequences=nseq, row_capacity=cfg.max_packed_len)
            bid = self._batch_id()
            yield AssembledBatch(bid, arrays, stats,
                                 self._lineage(bid, items, "pack", {"rows": R, "padding_ratio": stats.padding_ratio}), len(items))


def create_batch_assembler(cfg: BatchConfig, packed: bool = True, start_batch_index: int = 0):
    return (SequencePackedBatchAssembler if packed else PaddedBatchAssembler)(cfg, start_batch_index)


def summarize_padding_stats(stats: Sequence[PaddingStats]) -> dict:
    """Aggregate over the micro-batches of one optimizer step (what the step's metrics report)."""
    if not stats:
        return {}
    valid = sum(s.valid_tokens for s in stats)
    cap = sum(s.capacity_tokens for s in stats)
    return {"padding_ratio": 1.0 - valid / cap, "valid_tokens": valid, "capacity_tokens": cap,
            "max_row_imbalance": max(s.row_imbalance for s in stats),
            "sequences": int(sum(int(s.row_num_sequences.sum()) for s in stats))}
