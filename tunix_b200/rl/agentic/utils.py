"""Agentic helpers: `RolloutSyncLock` (many rollouts / one weight sync, sync preferred;
tunix/rl/agentic/utils.py:238-283) and exact-token-continuity helpers (:296-335)."""
from __future__ import annotations

import contextlib
import threading

import numpy as np


class RolloutSyncLock:
    """Readers = in-flight rollouts, writer = weight sync. A waiting sync blocks new rollouts (sync preference)."""

    def __init__(self):
        self._cond = threading.Condition()
        self._rollouts = 0
        self._syncing = False
        self._sync_waiting = 0

    @contextlib.contextmanager
    def acquire_rollout(self):
        with self._cond:
            while self._syncing or self._sync_waiting > 0:
                self._cond.wait()
            self._rollouts += 1
        try:
            yield
        finally:
            with self._cond:
                self._rollouts -= 1
                self._cond.notify_all()

    @contextlib.contextmanager
    def acquire_weight_sync(self):
        with self._cond:
            self._sync_waiting += 1
            while self._rollouts > 0 or self._syncing:
                self._cond.wait()
            self._sync_waiting -= 1
            self._syncing = True
        try:
            yield
        finally:
            with self._cond:
                self._syncing = False
                self._cond.notify_all()

    @property
    def active_rollouts(self) -> int:
        return self._rollouts


def concat_conversation(prompt_tokens, steps) -> tuple:
    """Flatten a multi-turn episode into (conversation tokens, masks, logprobs): assistant tokens have mask 1 and
    their sampled log-probs, environment tokens mask 0 / logprob 0. Later turns reuse the recorded ids verbatim
    (exact token continuity: nothing is re-tokenised)."""
    toks, masks, lps = [], [], []
    for s in steps:
        if s.assistant_tokens is not None:
            a = np.asarray(s.assistant_tokens)
            toks.append(a)
            masks.append(np.ones_like(a) if s.assistant_masks is None else np.asarray(s.assistant_masks))
            lps.append(np.zeros(len(a), np.float32) if s.logprobs is None else np.asarray(s.logprobs, np.float32))
        if s.env_tokens is not None and len(s.env_tokens):
            e = np.asarray(s.env_tokens)
            toks.append(e)
            masks.append(np.zeros_like(e))
            lps.append(np.zeros(len(e), np.float32))
    if not toks:
        return np.zeros(0, np.int64), np.zeros(0, np.int32), np.zeros(0, np.float32)
    return np.concatenate(toks).astype(np.int64), np.concatenate(masks).astype(np.int32), np.concatenate(lps)
