"""Hosts the frozen reference, critic and reward models (tunix/rl/inference/inference_worker.py:22-102)."""
from __future__ import annotations

import torch

from .. import common


class InferenceWorker:
    def __init__(self, models: dict):
        for k in models:
            if k not in ("critic", "reference", "reward"):
                raise ValueError(f"Model role {k} is not supported. Supported: critic, reference, reward")
        self._models = models

    def get_model(self, role: str):
        if role not in self._models:
            raise ValueError(f"{role} model is not available")
        return self._models[role]

    @torch.no_grad()
    def get_ref_per_token_logps(self, prompt_tokens, completion_tokens, pad_id, eos_id, completion_mask=None,
                                temperature=None, chunk_size: int = 0, **kw):
        ref = self.get_model("reference")
        return common.compute_per_token_logps(ref, prompt_tokens, completion_tokens, pad_id, eos_id,
                                              completion_mask=completion_mask, stop_gradient=True,
                                              temperature=temperature, chunk_size=chunk_size, **kw)

    @torch.no_grad()
    def get_values(self, prompt_tokens, completion_tokens, pad_id, eos_id, completion_mask=None):
        critic = self.get_model("critic")
        out = common.compute_score(critic, prompt_tokens, completion_tokens, pad_id, eos_id)
        out = out[0] if isinstance(out, tuple) else out
        P = prompt_tokens.shape[1]
        v = out[:, P - 1:-1]
        return v[..., 0] if v.dim() == 3 else v

    @torch.no_grad()
    def get_rewards(self, prompt_tokens, completion_tokens, pad_id, eos_id, completion_mask=None):
        """Score at the last real token of every sequence."""
        rm = self.get_model("reward")
        out = common.compute_score(rm, prompt_tokens, completion_tokens, pad_id, eos_id)
        out = out[0] if isinstance(out, tuple) else out
        scores = out[..., 0] if out.dim() == 3 else out
        _, mask, _ = common.process_ids(prompt_tokens, completion_tokens, pad_id, eos_id, completion_mask)
        last = (mask.shape[1] - 1) - torch.flip(mask, dims=[1]).float().argmax(dim=1)
        return scores.gather(1, last[:, None])[:, 0]
