"""Mock rollout engine for tests and pipeline benchmarks (tunix/rl/rollout/mock_rollout.py:40-345):
random completions with configurable length distribution and simulated latency."""
from __future__ import annotations

import time
from typing import Optional

import numpy as np

from .base_rollout import BaseRollout, RolloutOutput


class MockRollout(BaseRollout):
    def __init__(self, tokenizer=None, vocab_size: int = 256, latency_s: float = 0.0, per_token_latency_s: float = 0.0,
                 length_distribution: str = "uniform", min_length: int = 1, seed: int = 0, model=None, pad_id: int = 0,
                 eos_id: int = 1):
        self._tok, self._vocab, self._lat, self._ptl = tokenizer, vocab_size, latency_s, per_token_latency_s
        self._dist, self._min, self._rng, self._model = length_distribution, min_length, np.random.default_rng(seed), model
        self._pad, self._eos = pad_id, eos_id
        self.updates = 0
        self.calls = 0

    def _length(self, max_len: int) -> int:
        if self._dist == "fixed":
            return max_len
        if self._dist == "geometric":
            return int(min(max_len, max(self._min, self._rng.geometric(4.0 / max(max_len, 4)))))
        return int(self._rng.integers(self._min, max_len + 1))

    def generate(self, prompts, rollout_config, **kwargs) -> RolloutOutput:
        self.calls += 1
        tok_prompts = kwargs.get("prompt_token_ids")
        n = len(tok_prompts) if tok_prompts is not None else len(prompts)
        max_len = rollout_config.max_tokens_to_generate
        tokens, logps, texts = [], [], []
        for _ in range(n):
            ln = self._length(max_len)
            t = self._rng.integers(2, self._vocab, ln).astype(np.int64)
            if ln < max_len:
                t[-1] = self._eos
            tokens.append(t)
            logps.append(-self._rng.random(ln).astype(np.float32))
            texts.append(self._tok.decode(t.tolist()) if self._tok is not None else " ".join(map(str, t.tolist())))
        if self._lat or self._ptl:
            time.sleep(self._lat + self._ptl * max(len(t) for t in tokens))
        P = rollout_config.max_prompt_length
        prm = np.full((n, P), self._pad, np.int64)
        lens = np.zeros(n, np.int64)
        for i in range(n):
            ids = list(tok_prompts[i]) if tok_prompts is not None else (
                self._tok.encode(prompts[i]) if self._tok is not None else [2 + (ord(c) % 50) for c in prompts[i]])
            ids = ids[-P:]
            prm[i, P - len(ids):] = ids
            lens[i] = len(ids)
        return RolloutOutput(text=texts, logits=None, tokens=tokens, left_padded_prompt_tokens=prm, logprobs=logps,
                             prompt_lengths=lens)

    def get_per_token_logps(self, prompt_tokens, completion_tokens, completion_mask=None):
        import torch
        return torch.zeros(completion_tokens.shape, dtype=torch.float32, device=completion_tokens.device)

    def update_params(self, params, filter_types=None) -> None:
        self.updates += 1

    def pad_id(self) -> int:
        return self._pad

    def eos_id(self) -> int:
        return self._eos

    def model(self):
        return self._model
