"""DPO / ORPO trainer on top of PeftTrainer (tunix/sft/dpo/dpo_trainer.py:194-798).

* inputs: raw strings (`DataInput`: prompts / chosen / rejected, tokenised here: prompts left-padded to
  `max_prompt_length`, responses right-padded to `max_response_length`, :700-788) or pre-tokenised
  (`TrainingInput`);
* chosen and rejected rows are concatenated on the batch axis so the policy runs ONE forward (:356-369);
* reference log-probs are computed in `_prepare_inputs` with the frozen reference model, or with the
  policy's own backbone with adapters disabled when the policy is a LoRA model (:389-401);
* DPO: -[log sigma(beta*Delta)(1-ls) + log sigma(-beta*Delta) ls], Delta = (logp_c - ref_c) - (logp_r - ref_r);
  ORPO: SFT NLL + lambda * odds-ratio loss, optional prompt loss and length averaging (:481-628);
* sequence log-prob = masked sum of per-token log-probs of the response, computed with the fused lm_head
  log-prob kernel (no [B, T, V] logits).
"""
from __future__ import annotations

import dataclasses
from typing import Any, Optional

import numpy as np
import torch
import torch.nn.functional as F

from ...common.configs import TrainingConfig
from ...lora import disable_adapters, is_lora_enabled
from ..peft_trainer import PeftTrainer
from ..utils import LossOutput, WeightedMetric


@dataclasses.dataclass(kw_only=True)
class DPOTrainingConfig(TrainingConfig):
    algorithm: str = "dpo"                 # "dpo" | "orpo"
    beta: float = 0.1
    lambda_orpo: float = 0.1
    label_smoothing: float = 0.0
    enable_prompt_loss_orpo: bool = True
    average_log_prob_orpo: bool = True
    max_prompt_length: Optional[int] = None
    max_response_length: Optional[int] = None

    def __post_init__(self):
        if self.algorithm not in ("dpo", "orpo"):
            raise ValueError(f"algorithm must be 'dpo' or 'orpo', got {self.algorithm!r}")
        if not 0.0 <= self.label_smoothing < 0.5:
            raise ValueError("label_smoothing must be in [0, 0.5)")


@dataclasses.dataclass
class DataInput:
    """Raw text triple(s)."""
    prompts: list
    chosen_responses: list
    rejected_responses: list


@dataclasses.dataclass
class TrainingInput:
    """Tokenised: prompt_ids [B,P] left-padded, chosen/rejected ids [B,R] right-padded, with masks."""
    prompt_ids: Any
    prompt_mask: Any
    chosen_ids: Any
    chosen_mask: Any
    rejected_ids: Any
    rejected_mask: Any


@dataclasses.dataclass
class TrainExample:
    input_ids: torch.Tensor            # [2B, P+R]  (chosen rows, then rejected rows)
    positions: torch.Tensor
    segment_ids: torch.Tensor          # 1 = real token, 0 = padding
    completion_mask: torch.Tensor      # [2B, R]
    logits_to_keep: int
    ref_chosen_logps: Optional[torch.Tensor] = None
    ref_rejected_logps: Optional[torch.Tensor] = None
    full_mask: Optional[torch.Tensor] = None


def compute_logps(model, input_ids, positions, segment_ids, logits_to_keep: int, completion_mask,
                  enable_prompt_loss: bool = False, full_mask=None):
    """Returns (chosen_logps [B], rejected_logps [B], prompt+chosen logps [B] | None)."""
    hidden, _ = model(input_ids, positions=positions, segment_ids=segment_ids, skip_lm_head=True)
    if enable_prompt_loss and full_mask is not None:
        lp_all, _ = model.token_logprobs(hidden[:, :-1], input_ids[:, 1:])
        lp = lp_all[:, -logits_to_keep:]
    else:
        lp_all = None
        lp, _ = model.token_logprobs(hidden[:, -logits_to_keep - 1:-1], input_ids[:, -logits_to_keep:])
    seq = (lp * completion_mask.float()).sum(-1)
    B = seq.shape[0] // 2
    prompt_chosen = None
    if lp_all is not None:
        prompt_chosen = (lp_all[:B] * full_mask[:B, 1:].float()).sum(-1)
    return seq[:B], seq[B:], prompt_chosen


def dpo_loss_fn(model, train_example: TrainExample, algorithm: str = "dpo", beta: float = 0.1,
                lambda_orpo: float = 0.1, label_smoothing: float = 0.0, enable_prompt_loss_orpo: bool = False,
                average_log_prob_orpo: bool = False) -> LossOutput:
    ex = train_example
    chosen, rejected, prompt_chosen = compute_logps(
        model, ex.input_ids, ex.positions, ex.segment_ids, ex.logits_to_keep, ex.completion_mask,
        enable_prompt_loss=(algorithm == "orpo" and enable_prompt_loss_orpo), full_mask=ex.full_mask)
    B = ex.completion_mask.shape[0] // 2
    denom = torch.tensor(float(B), device=chosen.device)
    wm = lambda x: WeightedMetric(x.detach().sum(), denom, min_denominator=1.0)  # noqa: E731
    ls = label_smoothing
    if algorithm == "orpo":
        cm, rm = ex.completion_mask[:B].float(), ex.completion_mask[B:].float()
        if average_log_prob_orpo:
            chosen = chosen / cm.sum(-1).clamp(min=1.0)
            rejected = rejected / rm.sum(-1).clamp(min=1.0)
        if enable_prompt_loss_orpo and prompt_chosen is not None:
            sft = -prompt_chosen / ex.full_mask[:B, 1:].float().sum(-1).clamp(min=1.0) if average_log_prob_orpo \
                else -prompt_chosen
        else:
            sft = -chosen
        eps = 1e-7
        c, r = chosen.clamp(max=-eps), rejected.clamp(max=-eps)
        log_odds = (c - r) - (torch.log1p(-torch.exp(c)) - torch.log1p(-torch.exp(r)))
        or_loss = -(F.logsigmoid(log_odds) * (1 - ls) + F.logsigmoid(-log_odds) * ls)
        total = sft + lambda_orpo * or_loss
        cr, rr = lambda_orpo * c, lambda_orpo * r
        aux = {"rewards/chosen": wm(cr), "rewards/rejected": wm(rr), "rewards/margin": wm(cr - rr),
               "rewards/accuracy": wm((cr > rr).float()), "log_probs/chosen": wm(c), "log_probs/rejected": wm(r),
               "odds_ratio": wm(torch.exp(log_odds)), "sft_loss": wm(sft), "or_loss": wm(or_loss)}
        return LossOutput(WeightedMetric(total.sum(), denom, min_denominator=1.0), aux)
    c_ratio = chosen - ex.ref_chosen_logps if ex.ref_chosen_logps is not None else chosen
    r_ratio = rejected - ex.ref_rejected_logps if ex.ref_rejected_logps is not None else rejected
    delta = c_ratio - r_ratio
    losses = -(F.logsigmoid(beta * delta) * (1 - ls) + F.logsigmoid(-beta * delta) * ls)
    cr, rr = beta * c_ratio, beta * r_ratio
    aux = {"rewards/chosen": wm(cr), "rewards/rejected": wm(rr), "rewards/margin": wm(cr - rr),
           "rewards/accuracy": wm((cr > rr).float()), "log_probs/chosen": wm(chosen), "log_probs/rejected": wm(rejected)}
    return LossOutput(WeightedMetric(losses.sum(), denom, min_denominator=1.0), aux)


def _pad(rows, length: int, pad_id: int, left: bool):
    ids = np.full((len(rows), length), pad_id, np.int64)
    mask = np.zeros((len(rows), length), np.int32)
    for i, r in enumerate(rows):
        r = list(r)
        r = r[-length:] if left else r[:length]
        if left:
            ids[i, length - len(r):], mask[i, length - len(r):] = r, 1
        else:
            ids[i, :len(r)], mask[i, :len(r)] = r, 1
    return ids, mask


class DPOTrainer(PeftTrainer):
    def __init__(self, model, ref_model, optimizer, training_config: DPOTrainingConfig, tokenizer=None,
                 metrics_logger=None):
        super().__init__(model, optimizer, training_config, metrics_logger)
        self.ref_model = ref_model
        self.tokenizer = tokenizer
        self.dpo_config = training_config
        self._share_backbone = ref_model is None and is_lora_enabled(model)
        cfg = training_config
        self.with_loss_fn(lambda m, train_example: dpo_loss_fn(
            m, train_example, cfg.algorithm, cfg.beta, cfg.lambda_orpo, cfg.label_smoothing,
            cfg.enable_prompt_loss_orpo, cfg.average_log_prob_orpo), has_aux=True)
        self.with_gen_model_input_fn(lambda ex: {"train_example": ex})

    def _tokenize(self, d: DataInput) -> TrainingInput:
        if self.tokenizer is None:
            raise ValueError("a tokenizer is required for string inputs")
        cfg = self.dpo_config
        if cfg.max_prompt_length is None or cfg.max_response_length is None:
            raise ValueError("max_prompt_length and max_response_length must be set for string inputs")
        tok, pad = self.tokenizer, self.tokenizer.pad_id()
        eos = tok.eos_id()
        p = [tok.encode(s) for s in d.prompts]
        bos = tok.bos_id()
        if bos is not None:
            p = [[bos] + x if (not x or x[0] != bos) else x for x in p]
        c = [tok.encode(s) + [eos] for s in d.chosen_responses]
        r = [tok.encode(s) + [eos] for s in d.rejected_responses]
        pi, pm = _pad(p, cfg.max_prompt_length, pad, left=True)
        ci, cm = _pad(c, cfg.max_response_length, pad, left=False)
        ri, rm = _pad(r, cfg.max_response_length, pad, left=False)
        return TrainingInput(pi, pm, ci, cm, ri, rm)

    def _shard_and_move(self, batch):
        return batch   # TrainExample tensors are already on the device and local (see _prepare_inputs)

    @torch.no_grad()
    def _prepare_inputs(self, batch: Any) -> TrainExample:
        from .. import sharding_utils
        if isinstance(batch, TrainExample):
            return batch
        if isinstance(batch, DataInput):
            batch = self._tokenize(batch)
        batch = sharding_utils.shard_input(batch, self.config.data_sharding_axis)
        dev = self.device
        t = lambda a: torch.as_tensor(np.asarray(a) if not isinstance(a, torch.Tensor) else a).to(dev)  # noqa: E731
        pi, pm = t(batch.prompt_ids).long(), t(batch.prompt_mask).to(torch.int32)
        ci, cm = t(batch.chosen_ids).long(), t(batch.chosen_mask).to(torch.int32)
        ri, rm = t(batch.rejected_ids).long(), t(batch.rejected_mask).to(torch.int32)
        input_ids = torch.cat([torch.cat([pi, ci], 1), torch.cat([pi, ri], 1)], 0)
        full_mask = torch.cat([torch.cat([pm, cm], 1), torch.cat([pm, rm], 1)], 0)
        positions = torch.clamp(torch.cumsum(full_mask, -1) - 1, min=0).to(torch.int32)
        completion_mask = torch.cat([cm, rm], 0)
        R = ci.shape[1]
        ex = TrainExample(input_ids=input_ids, positions=positions, segment_ids=full_mask,
                          completion_mask=completion_mask, logits_to_keep=R, full_mask=full_mask)
        if self.dpo_config.algorithm == "dpo" and (self.ref_model is not None or self._share_backbone):
            if self._share_backbone:
                with disable_adapters(self.model):
                    rc, rr, _ = compute_logps(self.model, input_ids, positions, full_mask, R, completion_mask)
            else:
                rc, rr, _ = compute_logps(self.ref_model, input_ids, positions, full_mask, R, completion_mask)
            ex.ref_chosen_logps, ex.ref_rejected_logps = rc.detach(), rr.detach()
        return ex


DpoTrainer = DPOTrainer
ORPOTrainer = DPOTrainer
OrpoTrainer = DPOTrainer
DpoTrainingConfig = DPOTrainingConfig
ORPOTrainingConfig = DPOTrainingConfig
OrpoTrainingConfig = DPOTrainingConfig
