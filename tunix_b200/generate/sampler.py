"""`Sampler`: prefill + decode loop over a dense contiguous KV cache (the "vanilla" rollout engine).

API and behaviour follow tunix/generate/sampler.py:205-1080: left-padded prompts bucketed to a power of
two, greedy / temperature+top-p(+top-k) / beam search, per-step RNG derived from (seed, step), forbidden
tokens, multi-EOS stop, optional per-token log-probs and logits, echo, padded or ragged outputs, token-id
prompts, `update_params` (full or LoRA-only). Left padding is expressed with segment ids (pad = 0), so the
flash-attention kernels mask it without a dense [T, S] mask.

The GPU fast path for RL rollouts is `generate/engine.py` (paged KV, CUDA-graphed decode); this class is
the reference-compatible engine that runs anywhere the model runs, CPU included.
"""
from __future__ import annotations

import math
from typing import Any, Iterable, Optional, Sequence

import numpy as np
import torch

from ..common.configs import CacheConfig
from . import beam_search as beam_lib
from . import sampling
from .base_sampler import BaseSampler, SamplerOutput


def next_power_of_2(x: int) -> int:
    return 1 if x <= 1 else 2 ** math.ceil(math.log2(x))


def pad_prompts_left(token_rows: Sequence[Sequence[int]], length: int, pad_id: int) -> tuple[np.ndarray, np.ndarray]:
    out = np.full((len(token_rows), length), pad_id, np.int64)
    lens = np.zeros(len(token_rows), np.int64)
    for i, row in enumerate(token_rows):
        row = list(row)[-length:]
        out[i, length - len(row):] = row
        lens[i] = len(row)
    return out, lens


class Sampler(BaseSampler):
    def __init__(self, transformer, tokenizer, cache_config: CacheConfig):
        self._model = transformer
        self.tokenizer = tokenizer
        self.cache_config = cache_config
        self.device = next(transformer.parameters()).device
        self.dtype = next(transformer.parameters()).dtype

    @property
    def transformer(self):
        return self._model

    @property
    def transformer_state(self):
        return dict(self._model.named_parameters())

    def tokenize(self, input_string: str):
        ids = self.tokenizer.encode(input_string)
        bos = self.tokenizer.bos_id()
        if bos is not None and (not ids or ids[0] != bos):
            ids = [bos] + list(ids)
        return np.asarray(ids, np.int64)

    @torch.no_grad()
    def update_params(self, updated_weights: dict, filter_types=None) -> None:
        """Copy weights (full or LoRA-only dict name -> tensor) into the sampler's model, casting dtype."""
        own = dict(self._model.named_parameters())
        for name, w in updated_weights.items():
            if name not in own:
                raise KeyError(f"unknown parameter {name!r} in weight update")
            if own[name].data_ptr() == w.data_ptr():
                continue  # shared storage: nothing to do
            own[name].copy_(w.to(own[name].device, own[name].dtype))

    # ------------------------------------------------------------------ call
    @torch.no_grad()
    def __call__(self, input_strings=None, max_generation_steps: int = 0, max_prompt_length: Optional[int] = None,
                 echo: bool = False, return_logits: bool = False, return_logprobs: bool = False,
                 eos_tokens: Optional[Sequence[int]] = None, forbidden_tokens: Optional[Iterable[int]] = None,
                 temperature: float = 0.0, top_p: Optional[float] = None, top_k: Optional[int] = None,
                 beam_size: Optional[int] = None, seed: Optional[int] = None, pad_output: bool = False, *,
                 prompt_token_ids: Optional[Sequence[Sequence[int]]] = None,
                 model_inputs: Optional[dict] = None, return_routed_experts: bool = False) -> SamplerOutput:
        """`model_inputs`: extra keyword tensors for the prefill pass of a multimodal model (e.g. `pixel_values`,
        `pixel_position_ids`, `input_features`): the prompts carry the placeholder tokens, the decode steps are
        text only (tunix/generate/sampler.py: images / audio hooks). `return_routed_experts`: for a mixture-of-experts
        model, also return per sequence the experts every token was routed to, `[prompt + completion - 1 or so,
        num_layers, top_k]` (prompt tokens, then one row per token that was fed back), for router replay in the
        trainer."""
        if (input_strings is None) == (prompt_token_ids is None):
            raise ValueError("give exactly one of input_strings / prompt_token_ids")
        if isinstance(input_strings, str):
            input_strings = [input_strings]
        rows = [list(r) for r in prompt_token_ids] if prompt_token_ids is not None else \
            [self.tokenize(s).tolist() for s in input_strings]
        eos_ids = list(eos_tokens) if eos_tokens else [self.tokenizer.eos_id()]
        pad_id = self.tokenizer.pad_id()
        longest = max(len(r) for r in rows)
        plen = max_prompt_length if max_prompt_length else next_power_of_2(longest)
        plen = max(plen, 1)
        total = plen + max_generation_steps
        if total > self.cache_config.cache_size:
            raise ValueError(f"prompt bucket {plen} + {max_generation_steps} steps exceeds cache size "
                             f"{self.cache_config.cache_size}")
        prompts, plens = pad_prompts_left(rows, plen, pad_id)
        if beam_size is not None and beam_size > 1:
            return self._beam(prompts, plens, max_generation_steps, beam_size, eos_ids, pad_id, echo, pad_output)
        dev = self.device
        B = prompts.shape[0]
        toks = torch.from_numpy(prompts).to(dev)
        valid = (toks != pad_id) | (torch.arange(plen, device=dev)[None] >= (plen - torch.from_numpy(plens).to(dev))[:, None])
        seg = valid.to(torch.int32)
        positions = torch.clamp(torch.cumsum(seg, -1) - 1, min=0).to(torch.int32)
        cache = self._model.init_cache(B, total, self.dtype, dev)
        was_training = self._model.training
        self._model.eval()
        extra = {k: (v.to(dev) if hasattr(v, "to") else v) for k, v in (model_inputs or {}).items()}
        hidden, cache = self._model(toks, positions=positions, cache=cache, segment_ids=seg, skip_lm_head=True, **extra)
        last_h = hidden[:, -1:]
        next_pos = positions[:, -1:] + 1
        routed_steps = None
        if return_routed_experts and hasattr(self._model, "routed_experts_of_last_forward"):
            r0 = self._model.routed_experts_of_last_forward()
            routed_steps = [r0] if r0 is not None else None           # [B, plen, L, k], left-padded like the prompt
        forbidden = torch.as_tensor(sorted(set(forbidden_tokens)), device=dev) if forbidden_tokens else None
        eos_t = torch.as_tensor(eos_ids, device=dev)
        out_tokens = torch.full((B, max_generation_steps), pad_id, dtype=torch.long, device=dev)
        out_logps = torch.zeros((B, max_generation_steps), dtype=torch.float32, device=dev) if return_logprobs else None
        out_logits = [] if return_logits else None
        done = torch.zeros(B, dtype=torch.bool, device=dev)
        seed = 0 if seed is None else int(seed)
        n_steps = 0
        ones = torch.ones(B, 1, dtype=torch.int32, device=dev)
        for step in range(max_generation_steps):
            logits = self._model.compute_final_logits(last_h)[:, 0].float()
            if forbidden is not None:
                logits[:, forbidden] = -float("inf")
            tok, logp = sampling.sample(logits, temperature=temperature, top_p=top_p, top_k=top_k, seed=seed, step=step,
                                        want_logprob=return_logprobs)
            tok = torch.where(done, torch.full_like(tok, pad_id), tok)
            out_tokens[:, step] = tok
            if return_logprobs:
                out_logps[:, step] = torch.where(done, torch.zeros_like(logp), logp)
            if return_logits:
                out_logits.append(logits)
            done = done | (tok.unsqueeze(-1) == eos_t).any(-1)
            n_steps = step + 1
            if bool(done.all()):
                break
            hidden, cache = self._model(tok[:, None], positions=next_pos, cache=cache, segment_ids=ones,
                                        skip_lm_head=True)
            last_h = hidden
            next_pos = next_pos + 1
            if routed_steps is not None:
                routed_steps.append(self._model.routed_experts_of_last_forward())
        self._model.train(was_training)
        out = self._finish(prompts, plens, out_tokens[:, :max(n_steps, 0)], out_logps, out_logits, eos_ids, pad_id, echo,
                           pad_output, max_generation_steps)
        if routed_steps is not None:
            allr = torch.cat(routed_steps, 1).to(torch.int16).cpu().numpy()          # [B, plen + fed tokens, L, k]
            P = prompts.shape[1]
            # per sequence: its real prompt tokens, then the completion tokens that were fed back (all but the last)
            out.routed_experts = [allr[b, P - int(plens[b]):P + max(len(out.tokens[b]) - (len(prompts[b]) if echo else 0) - 1, 0)]
                                  for b in range(B)]
        return out

    # ------------------------------------------------------------ post-process
    def _finish(self, prompts, plens, gen: torch.Tensor, logps, logits, eos_ids, pad_id, echo, pad_output, max_steps):
        gen_np = gen.cpu().numpy()
        B = gen_np.shape[0]
        tokens, texts, lp_out = [], [], [] if logps is not None else None
        lp_np = logps.cpu().numpy() if logps is not None else None
        for b in range(B):
            row = gen_np[b]
            stop = len(row)
            for i, t in enumerate(row):
                if t in eos_ids:
                    stop = i + 1
                    break
            row = row[:stop]
            text_ids = [t for t in row if t not in eos_ids and t != pad_id]
            if echo:
                prm = prompts[b, prompts.shape[1] - plens[b]:]
                row = np.concatenate([prm, row])
                text_ids = list(prm) + text_ids
            if pad_output:
                width = max_steps + (prompts.shape[1] if echo else 0)
                row = np.concatenate([row, np.full(width - len(row), pad_id, row.dtype)])
            tokens.append(row)
            texts.append(self.tokenizer.decode(text_ids))
            if lp_np is not None:
                lp_out.append(lp_np[b, :stop].tolist())
        tok_out = np.stack(tokens) if pad_output else tokens
        lg = torch.stack(logits, 1) if logits else None
        return SamplerOutput(text=texts, logits=lg, tokens=tok_out, padded_prompt_tokens=prompts, logprobs=lp_out,
                             prompt_lengths=np.asarray(plens))

    def _beam(self, prompts, plens, max_steps, beam_size, eos_ids, pad_id, echo, pad_output):
        gen = beam_lib.beam_search(self._model, prompts, plens, max_steps, beam_size, eos_ids, pad_id, self.dtype,
                                   self.device)
        return self._finish(prompts, plens, gen, None, None, eos_ids, pad_id, echo, pad_output, max_steps)
