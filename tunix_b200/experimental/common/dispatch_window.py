"""Bounded-staleness dispatch of prompt batches (tunix/experimental/common/dispatch_window.py:26-214).

The dispatcher may hand out prompts of batch `b` while `b <= next_batch + max_staleness`, where `next_batch` is
the batch the trainer will consume next; beyond that `wait_for(b)` parks until `release()`. Groups that a filter
dropped count towards the window (every `full_batch_size` dropped groups move it by one batch, so replacements
can be dispatched), and for out-of-order resume the ids of the prompts that were trained on or skipped are kept
as checkpoint metadata, so a restart skips exactly those."""
from __future__ import annotations

import asyncio
from typing import Callable, Mapping, Optional, Sequence


def _prompt_id(item) -> Optional[str]:
    if isinstance(item, Mapping):
        pid = item.get("prompt_id")
    else:
        pid = getattr(item, "prompt_id", None)
    return str(pid) if pid not in (None, "") else None


class DispatchWindow:
    def __init__(self, max_staleness: int, next_batch_fn: Callable[[], int], *, full_batch_size: int = 1,
                 out_of_order_resume: bool = False):
        if max_staleness < 0:
            raise ValueError(f"max_staleness must be non-negative, got {max_staleness}")
        if full_batch_size <= 0:
            raise ValueError(f"full_batch_size must be positive, got {full_batch_size}")
        self.max_staleness, self.full_batch_size = max_staleness, full_batch_size
        self.out_of_order_resume = out_of_order_resume
        self._next_batch_fn = next_batch_fn
        self._release = asyncio.Event()
        self._filtered_groups = 0
        self.committed_prompt_ids: set = set()
        self.skipped_prompt_ids: set = set()
        self._resumed = False

    @property
    def next_batch(self) -> int:
        return self._next_batch_fn() + -(-self._filtered_groups // self.full_batch_size)

    @property
    def uses_prompt_id_resume(self) -> bool:
        return self.out_of_order_resume and self._resumed

    @property
    def dataset_skip_count(self) -> int:
        """Prompts to skip at the head of the dataset on restart (0 when resume goes by prompt id)."""
        return 0 if self.uses_prompt_id_resume else self.next_batch * self.full_batch_size

    def release(self) -> None:
        self._release.set()

    def on_group_filtered(self, group: Sequence) -> None:
        pid = _prompt_id(group[0]) if group else None
        if pid:
            self.skipped_prompt_ids.add(pid)
        self._filtered_groups += 1
        self.release()

    def record_committed_groups(self, groups: Sequence[Sequence]) -> None:
        if self.out_of_order_resume:
            self.committed_prompt_ids.update(p for g in groups if g for p in [_prompt_id(g[0])] if p)

    def checkpoint_metadata(self, pending_groups: Sequence[Sequence] = ()) -> dict:
        if not self.out_of_order_resume or (self.max_staleness <= 0 and not self.skipped_prompt_ids and not self._resumed):
            return {}
        pending = {p for g in pending_groups if g for p in [_prompt_id(g[0])] if p}
        return {"committed_prompt_ids": sorted(self.committed_prompt_ids | pending),
                "skipped_prompt_ids": sorted(self.skipped_prompt_ids)}

    def restore_checkpoint_metadata(self, meta) -> bool:
        if not self.out_of_order_resume or not isinstance(meta, Mapping) or not (
                "committed_prompt_ids" in meta or "skipped_prompt_ids" in meta):
            return False

        def ids(key):
            raw = meta.get(key, ())
            return {str(p) for p in raw} if isinstance(raw, Sequence) and not isinstance(raw, (str, bytes)) else set()
        self._resumed = True
        self.committed_prompt_ids, self.skipped_prompt_ids = ids("committed_prompt_ids"), ids("skipped_prompt_ids")
        return True

    async def wait_for(self, batch_idx: int) -> None:
        while batch_idx > self.next_batch + self.max_staleness:
            # wait first, clear second: the other order can lose a release that lands between test and clear
            await self._release.wait()
            self._release.clear()

    def admit(self, prompt_item) -> bool:
        """False for a prompt that a restored run has already trained on or skipped."""
        if not self.uses_prompt_id_resume:
            return True
        pid = _prompt_id(prompt_item)
        return pid is None or (pid not in self.committed_prompt_ids and pid not in self.skipped_prompt_ids)
