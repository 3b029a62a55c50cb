"""Rollout on the in-framework sampler (tunix/rl/rollout/vanilla_rollout.py:31-106)."""
from __future__ import annotations

import numpy as np

from ...common.configs import CacheConfig, RolloutConfig
from ...generate.sampler import Sampler
from .. import common
from .base_rollout import BaseRollout, RolloutOutput


def _page_budget(model, cache_size: int, rc: RolloutConfig):
    """Pages of the KV pool: enough for `max_running_requests` full-length sequences, but no more than
    `hbm_utilization` of the device memory that is free when the engine is built (requests that find no page wait in
    the engine's queue). None (= the engine's own sizing) off the GPU."""
    import torch
    cfg = model.config
    dev = next(model.parameters()).device
    per_seq = -(-int(cache_size) // int(rc.page_size))
    want = int(rc.max_running_requests) * per_seq
    if dev.type != "cuda" or not rc.hbm_utilization:
        return want
    page_bytes = cfg.num_layers * 2 * cfg.num_kv_heads * cfg.head_dim * int(rc.page_size) * 2
    free, _ = torch.cuda.mem_get_info(dev)
    cap = int(free * float(rc.hbm_utilization)) // max(page_bytes, 1)
    return max(min(want, cap), per_seq)             # never below one full sequence


class VanillaRollout(BaseRollout):
    def __init__(self, model, tokenizer, cache_config_or_size, engine: str = "dense", rollout_config: RolloutConfig = None):
        """`rollout_config` (paged engine): its `page_size`, `max_running_requests`, `use_cuda_graph` and
        `chunked_prefill_size` size the engine; without it the engine's own defaults apply."""
        cfg = model.config
        if isinstance(cache_config_or_size, int):
            cache_config_or_size = CacheConfig(cache_config_or_size, cfg.num_layers, cfg.num_kv_heads, cfg.head_dim)
        self._tokenizer = tokenizer
        self._sampler = Sampler(model, tokenizer, cache_config_or_size)
        self._engine = None
        if engine == "paged":
            from ...generate.engine import PagedEngine
            knobs = {}
            if rollout_config is not None:
                knobs = dict(page_size=int(rollout_config.page_size), max_running_requests=int(rollout_config.max_running_requests),
                             use_cuda_graph=bool(rollout_config.use_cuda_graph),
                             prefill_chunk=int(rollout_config.chunked_prefill_size or 0))
                knobs["num_pages"] = _page_budget(model, cache_config_or_size.cache_size, rollout_config)
            self._engine = PagedEngine(model, tokenizer, cache_config_or_size, **knobs)

    def generate(self, prompts, rollout_config: RolloutConfig, **kwargs) -> RolloutOutput:
        want_tp = getattr(rollout_config, "tensor_parallel_size", -1)
        have_tp = getattr(self._engine, "tpw", 1) if self._engine is not None else 1
        if want_tp not in (-1, 0, 1) and want_tp != have_tp:
            # tensor-parallel decode runs on a model that `parallel.tp.apply_tensor_parallel` has sliced over a group of
            # that size (paged engine only); every rank of the group must be handed the same requests
            raise NotImplementedError(f"RolloutConfig.tensor_parallel_size={want_tp}, but the rollout model is sliced over "
                                      f"{have_tp} rank(s): slice it with apply_tensor_parallel and use the paged engine")
        tok_prompts = kwargs.get("prompt_token_ids")
        call = self._engine if self._engine is not None else self._sampler
        extra = {}
        if self._engine is None and (getattr(rollout_config, "return_routed_experts", False)
                                     or getattr(rollout_config, "store_routed_experts", False)):
            extra["return_routed_experts"] = True        # dense sampler only: the paged engine does not record routing
        out = call(**extra, input_strings=None if tok_prompts is not None else prompts,
                   prompt_token_ids=tok_prompts,
                   max_generation_steps=rollout_config.max_tokens_to_generate,
                   max_prompt_length=rollout_config.max_prompt_length, temperature=rollout_config.temperature,
                   top_p=rollout_config.top_p, top_k=rollout_config.top_k, seed=rollout_config.seed,
                   eos_tokens=rollout_config.eos_tokens, return_logprobs=rollout_config.return_logprobs,
                   echo=False, pad_output=False)
        lps = [np.asarray(l, np.float32) for l in out.logprobs] if out.logprobs is not None else None
        return RolloutOutput(text=out.text, logits=None, tokens=[np.asarray(t) for t in out.tokens],
                             left_padded_prompt_tokens=out.padded_prompt_tokens, logprobs=lps,
                             routed_experts=out.routed_experts, prompt_lengths=out.prompt_lengths)

    def start_server(self, rollout_config: RolloutConfig):
        """Server mode of the paged engine (single requests join the running batch): the continuous-batching
        server the reference requires of vLLM for agentic rollouts (tunix/rl/agentic/agentic_rl_learner.py:293-301).
        None on the dense sampler."""
        if self._engine is None:
            return None
        from ...generate.engine import EngineServer
        rc = rollout_config
        return EngineServer(self._engine, max_new_tokens=rc.max_tokens_to_generate, max_prompt_length=rc.max_prompt_length,
                            temperature=rc.temperature, top_p=rc.top_p, top_k=rc.top_k, seed=rc.seed or 0,
                            eos_tokens=rc.eos_tokens)

    def get_per_token_logps(self, prompt_tokens, completion_tokens, completion_mask=None):
        return common.compute_per_token_logps(self.model(), prompt_tokens, completion_tokens, self.pad_id(), self.eos_id(),
                                              completion_mask=completion_mask, stop_gradient=True)

    def update_params(self, params, filter_types=None) -> None:
        self._sampler.update_params(params, filter_types)

    def pad_id(self) -> int:
        return self._tokenizer.pad_id()

    def eos_id(self) -> int:
        return self._tokenizer.eos_id()

    def model(self):
        return self._sampler.transformer
