"""Shared RL math: train-example container, per-token log-probs, KL, loss aggregation, sampler/trainer agreement.

Behaviour follows tunix/rl/common.py: `TrainExample` (:103-142), `compute_kl_divergence` (:145-204),
`selective_log_softmax` (:207-226), `process_ids` (:256-323), `compute_per_token_logps` (:415-606; here always
through the fused lm_head log-prob kernel, so the chunked and the full-logits path of the reference are the
same path), agreement / TIS / RS (:1002-1210), segmented sums (:1433-1489), `aggregate_loss` (:1492-1679).
All math in fp32 on whatever device the inputs live on.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Optional

import numpy as np
import torch

from ..sft.utils import WeightedMetric


@dataclasses.dataclass
class TrainExample:
    prompt_ids: torch.Tensor
    prompt_mask: torch.Tensor
    completion_ids: torch.Tensor
    completion_mask: torch.Tensor
    advantages: torch.Tensor                       # [B] unpacked, [B,T] packed / token-level
    ref_per_token_logps: Optional[torch.Tensor] = None
    old_per_token_logps: Optional[torch.Tensor] = None
    segment_ids: Optional[torch.Tensor] = None
    segment_positions: Optional[torch.Tensor] = None
    num_segments: Optional[int] = None
    is_update_step: Optional[bool] = None
    sampler_is_weights: Optional[torch.Tensor] = None
    routed_experts: Optional[torch.Tensor] = None
    sampler_agreement_applied: bool = False
    returns: Optional[torch.Tensor] = None          # PPO
    old_values: Optional[torch.Tensor] = None       # PPO
    policy_version: Optional[Any] = None


# -------------------------------------------------------------------------- KL
def compute_kl_divergence(per_token_logps, ref_per_token_logps, method: str = "kl", clamp: Optional[float] = None):
    new = torch.nan_to_num(per_token_logps.float(), nan=-100.0).clamp(-100.0, 100.0)
    ref = torch.nan_to_num(ref_per_token_logps.float(), nan=-100.0).clamp(-100.0, 100.0)
    if method == "kl":
        kl = new - ref
    elif method == "mse_kl":
        kl = 0.5 * (new - ref) ** 2
    elif method == "low_var_kl":
        d = (ref - new).clamp(-20.0, 20.0)
        kl = torch.exp(d) - d - 1.0
    else:
        raise ValueError(f"unknown KL method {method!r}")
    if clamp is not None:
        kl = kl.clamp(-clamp, clamp)
    return kl


def selective_log_softmax(logits: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """log_softmax(logits)[index] without a second full-vocab tensor."""
    lse = torch.logsumexp(logits.float(), dim=-1)
    picked = logits.float().gather(-1, index.long().unsqueeze(-1)).squeeze(-1)
    return picked - lse


# ------------------------------------------------------------------ id handling
def make_completion_mask(completion_ids: torch.Tensor, eos_tok) -> torch.Tensor:
    """1 up to and including the first EOS, 0 afterwards (multi-EOS aware)."""
    eos = torch.as_tensor(eos_tok if isinstance(eos_tok, (list, tuple)) else [eos_tok], device=completion_ids.device)
    is_eos = (completion_ids.unsqueeze(-1) == eos).any(-1)
    T = completion_ids.shape[1]
    first = torch.where(is_eos.any(1), is_eos.float().argmax(1), torch.full_like(is_eos[:, 0].long(), T))
    return (torch.arange(T, device=completion_ids.device)[None] <= first[:, None]).to(torch.int32)


def pad_to_length(x: torch.Tensor, length: int, pad_value=0, left: bool = False, dim: int = -1) -> torch.Tensor:
    n = x.shape[dim]
    if n >= length:
        return x
    shape = list(x.shape)
    shape[dim] = length - n
    pad = torch.full(shape, pad_value, dtype=x.dtype, device=x.device)
    return torch.cat([pad, x] if left else [x, pad], dim=dim)


def build_positions_from_mask(mask: torch.Tensor) -> torch.Tensor:
    return torch.clamp(torch.cumsum(mask.to(torch.int32), -1) - 1, min=0).to(torch.int32)


def process_ids(prompt_tokens, completion_tokens, pad_id, eos_id, completion_mask=None):
    """Concatenate prompt and completion; build masks, positions and segment ids (pad = 0, real = 1)."""
    prompt_mask = (prompt_tokens != pad_id).to(torch.int32)
    if completion_mask is None:
        completion_mask = make_completion_mask(completion_tokens, eos_id) * (completion_tokens != pad_id)
    ids = torch.cat([prompt_tokens, completion_tokens], dim=1)
    mask = torch.cat([prompt_mask, (completion_mask > 0).to(torch.int32)], dim=1)
    positions = build_positions_from_mask(mask)
    return ids, mask, positions


def compute_per_token_logps(model, prompt_tokens, completion_tokens, pad_id, eos_id, *, completion_mask=None,
                            stop_gradient: bool = True, return_entropy: bool = False, segment_ids=None,
                            segment_positions=None, temperature: Optional[float] = None, chunk_size: int = 0,
                            token_mask=None, routed_experts=None):
    """log pi(completion_t | prompt, completion_<t) for every completion position -> [B, C] fp32 (and entropy).

    Packed inputs pass `segment_ids` / `segment_positions` over the concatenated row; otherwise validity comes
    from pad ids. The lm_head never materialises [B, T, V] logits."""
    P = prompt_tokens.shape[1]
    if segment_ids is not None:
        ids = torch.cat([prompt_tokens, completion_tokens], dim=1)
        seg = segment_ids
        positions = segment_positions if segment_positions is not None else build_positions_from_mask(seg > 0)
    else:
        ids, mask, positions = process_ids(prompt_tokens, completion_tokens, pad_id, eos_id, completion_mask)
        if token_mask is not None:
            mask = (token_mask > 0).to(torch.int32)
            positions = build_positions_from_mask(mask)
        seg = mask

    extra = {}
    if routed_experts is not None and getattr(getattr(model, "config", None), "is_moe", False):
        extra["routed_experts"] = torch.as_tensor(routed_experts, device=ids.device).long()

    def run():
        hidden, _ = model(ids, positions=positions, segment_ids=seg, skip_lm_head=True, **extra)
        if P > 0:
            h = hidden[:, P - 1:-1]
        else:
            # packed rows have no prompt side: token t is predicted from position t - 1, and nothing predicts the
            # first token of a row (it is a prompt token, masked out of every loss)
            h = torch.cat([torch.zeros_like(hidden[:, :1]), hidden[:, :-1]], dim=1)
        return model.token_logprobs(h, completion_tokens, temperature=temperature or 1.0,
                                    want_entropy=return_entropy, chunk=chunk_size or None)

    if stop_gradient:
        with torch.no_grad():
            logp, ent = run()
    else:
        logp, ent = run()
    return (logp, ent) if return_entropy else logp


UNSET_ROUTED_EXPERT = -1      # a router-replay slot the trainer leaves to the model's own router (0 is a real expert)


def align_routed_experts(routed_experts, completion_lengths, prompt_width: int, completion_width: int):
    """The sampler's routing, laid out over the trainer's padded `[prompt | completion]` stream.

    The sampler reports `[prompt_len + completion_len, num_layers, top_k]` per generation; the trainer sees prompts
    left-padded to `prompt_width` and completions right-padded to `completion_width`. Routing is padded the same
    way (over-long prompts keep their tail, over-long completions their head), so that every replayed expert stays
    with the token it was captured for; everything else is `UNSET_ROUTED_EXPERT`. Replay is all-or-nothing: one
    missing row and the batch falls back to the model's own router (returns None)
    (tunix/rl/common.py:331-393). Returns int16 `[B, prompt_width + completion_width, num_layers, top_k]`."""
    import numpy as np
    if not routed_experts or any(r is None for r in routed_experts):
        return None
    if len(routed_experts) != len(completion_lengths):
        raise ValueError(f"got {len(routed_experts)} routing rows but {len(completion_lengths)} completion lengths")
    rows = []
    for routed, clen in zip(routed_experts, completion_lengths):
        routed = np.asarray(routed, dtype=np.int16)
        if routed.ndim != 3:
            raise ValueError(f"routed_experts must be [length, num_layers, top_k]; got shape {routed.shape}")
        split = max(routed.shape[0] - int(clen), 0)
        p_part = routed[max(split - prompt_width, 0):split]
        c_part = routed[split:split + min(routed.shape[0] - split, completion_width)]
        row = np.full((prompt_width + completion_width,) + routed.shape[1:], UNSET_ROUTED_EXPERT, dtype=np.int16)
        row[prompt_width - p_part.shape[0]:prompt_width] = p_part
        row[prompt_width:prompt_width + c_part.shape[0]] = c_part
        rows.append(row)
    return np.stack(rows)


def get_per_token_logps(model, input_tokens, positions, segment_ids=None, logits_to_keep: Optional[int] = None):
    """Per-token log-probs of `input_tokens[:, 1:]` (tunix/rl/common.py:230-251)."""
    hidden, _ = model(input_tokens, positions=positions, segment_ids=segment_ids, skip_lm_head=True)
    h, tg = hidden[:, :-1], input_tokens[:, 1:]
    if logits_to_keep:
        h, tg = h[:, -logits_to_keep:], tg[:, -logits_to_keep:]
    return model.token_logprobs(h, tg)[0]


def compute_score(model, prompt_tokens, completion_tokens, pad_id, eos_id, stop_gradient: bool = True):
    """Scalar-head score per position for critic / reward models (tunix/rl/common.py:1303-1347)."""
    ids, mask, positions = process_ids(prompt_tokens, completion_tokens, pad_id, eos_id)

    def run():
        return model(ids, positions=positions, segment_ids=mask)

    if stop_gradient:
        with torch.no_grad():
            return run()
    return run()


# -------------------------------------------------------------- segmented sums
def segment_sum(values: torch.Tensor, segment_ids: torch.Tensor, num_segments: int) -> torch.Tensor:
    """Row-wise segment sums: [B,T] values, ids in [0, num_segments) -> [B, num_segments]."""
    out = torch.zeros(values.shape[0], num_segments, dtype=values.dtype, device=values.device)
    return out.scatter_add(1, segment_ids.long().clamp(0, num_segments - 1), values)


def _resolve_num_segments(segment_ids, num_segments):
    if segment_ids is None:
        return None
    if num_segments is None:
        num_segments = int(segment_ids.max().item()) + 1
    return num_segments


# ------------------------------------------------------------- loss aggregation
def aggregate_loss(per_token_loss: torch.Tensor, mask: torch.Tensor, mode: str, segment_ids=None,
                   num_segments: Optional[int] = None, norm: Optional[float] = None) -> WeightedMetric:
    """Reduce a [B,T] loss to (sum, denominator) so micro-batches combine exactly.

    Modes (tunix/rl/common.py:1492-1580): token-mean, sequence-mean-token-mean, sequence-mean-token-scale,
    seq-mean-token-sum, sequence-mean-token-sum-norm. With `segment_ids` a "sequence" is a segment (> 0) of a
    packed row instead of a row."""
    L = per_token_loss.float()
    m = mask.float()
    Lm = L * m
    if segment_ids is not None:
        S = _resolve_num_segments(segment_ids, num_segments)
        seq_sum = segment_sum(Lm, segment_ids, S)[:, 1:]
        seq_cnt = segment_sum(m, segment_ids, S)[:, 1:]
    else:
        seq_sum = Lm.sum(-1, keepdim=True)
        seq_cnt = m.sum(-1, keepdim=True)
    nonempty = (seq_cnt > 0).float()
    if mode == "token-mean":
        return WeightedMetric(Lm.sum(), m.sum(), min_denominator=1.0)
    if mode == "sequence-mean-token-mean":
        return WeightedMetric((seq_sum / seq_cnt.clamp(min=1.0)).sum(), nonempty.sum(), min_denominator=1.0)
    if mode == "sequence-mean-token-scale":
        if norm is None:
            if segment_ids is not None:
                raise ValueError("sequence-mean-token-scale needs an explicit `norm` with packed inputs")
            norm = float(per_token_loss.shape[-1])
        return WeightedMetric((seq_sum / norm).sum(), nonempty.sum(), min_denominator=1.0)
    if mode == "seq-mean-token-sum":
        return WeightedMetric(Lm.sum(), nonempty.sum(), min_denominator=1e-6)
    if mode == "sequence-mean-token-sum-norm":
        d = float(norm) if norm is not None else float(per_token_loss.shape[0])
        return WeightedMetric(Lm.sum(), torch.as_tensor(d, device=L.device), min_denominator=1e-6)
    raise ValueError(f"unknown loss aggregation mode {mode!r}")


def reduced_loss_agg(per_token_loss, mask, mode: str, segment_ids=None, num_segments=None, norm=None) -> torch.Tensor:
    """Independent eager reduction used as a logged cross-check of `aggregate_loss`."""
    L, m = per_token_loss.detach().float().cpu().numpy(), mask.detach().float().cpu().numpy()
    seqs = []
    if segment_ids is not None:
        sid = segment_ids.detach().cpu().numpy()
        for b in range(L.shape[0]):
            for s in np.unique(sid[b]):
                if s > 0:
                    sel = sid[b] == s
                    seqs.append((float((L[b][sel] * m[b][sel]).sum()), float(m[b][sel].sum())))
    else:
        seqs = [(float((L[b] * m[b]).sum()), float(m[b].sum())) for b in range(L.shape[0])]
    nonempty = [s for s in seqs if s[1] > 0]
    tot = float((L * m).sum())
    if mode == "token-mean":
        v = tot / max(float(m.sum()), 1.0)
    elif mode == "sequence-mean-token-mean":
        v = sum(s / max(c, 1.0) for s, c in seqs) / max(len(nonempty), 1.0)
    elif mode == "sequence-mean-token-scale":
        n = norm if norm is not None else L.shape[-1]
        v = sum(s / n for s, _ in seqs) / max(len(nonempty), 1.0)
    elif mode == "seq-mean-token-sum":
        v = tot / max(len(nonempty), 1e-6)
    elif mode == "sequence-mean-token-sum-norm":
        v = tot / max(norm if norm is not None else L.shape[0], 1e-6)
    else:
        raise ValueError(mode)
    return torch.tensor(v)


# ------------------------------------------------------ sampler/trainer agreement
def _pearson(x: torch.Tensor, y: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    n = w.sum().clamp(min=1.0)
    mx, my = (x * w).sum() / n, (y * w).sum() / n
    cov = ((x - mx) * (y - my) * w).sum()
    vx, vy = (((x - mx) ** 2) * w).sum(), (((y - my) ** 2) * w).sum()
    return cov / torch.sqrt(vx * vy).clamp(min=1e-20)


def _mean_op(vals):
    return float(np.mean([float(np.asarray(v)) for v in vals]))


def _max_op(vals):
    return float(np.max([float(np.asarray(v)) for v in vals]))


def _min_op(vals):
    return float(np.min([float(np.asarray(v)) for v in vals]))


def _sum_op(vals):
    return float(np.sum([float(np.asarray(v)) for v in vals]))


def sampler_trainer_agreement(rollout_per_token_logps, trainer_per_token_logps, completion_mask, sampler_is=None,
                              sampler_is_threshold: Optional[float] = 2.0, sampler_rs=None, sampler_rs_min=None,
                              sampler_rs_max=None, seq_logprob_error_threshold=None, segment_ids=None,
                              num_segments=None):
    """Sampler-vs-trainer log-prob agreement metrics, optional sequence error masking, truncated importance
    weights (`sampler_is`) and rejection gating (`sampler_rs`).

    Returns (metrics {name: (value, reducer)}, sampler_is_weights | None, filtered_completion_mask)."""
    metrics: dict = {}
    if rollout_per_token_logps is None or trainer_per_token_logps is None:
        return metrics, None, completion_mask
    if completion_mask is None:
        raise ValueError("Completion mask is required for sampler-trainer agreement metrics.")
    ro, tr = rollout_per_token_logps.float(), trainer_per_token_logps.detach().float()
    if ro.shape != tr.shape or ro.shape != completion_mask.shape:
        raise ValueError(f"Shape mismatch: rollout {tuple(ro.shape)}, trainer {tuple(tr.shape)}, mask {tuple(completion_mask.shape)}")
    mask_dtype = completion_mask.dtype
    mask = completion_mask > 0
    finite = torch.isfinite(ro) & torch.isfinite(tr)
    valid = mask & finite
    invalid_scored = mask & ~finite
    sro, strn = torch.where(valid, ro, 0.0), torch.where(valid, tr, 0.0)
    w = valid.float()
    n = w.sum().clamp(min=1.0)
    diff = (strn - sro).abs()
    mult_err = torch.where(valid, torch.exp(diff.clamp(max=20.0)), torch.zeros_like(diff))
    pro, ptr = torch.exp(sro) * w, torch.exp(strn) * w
    pdiff = (pro - ptr).abs()
    metrics.update({
        "sampler_trainer/logp_diff_mean": ((diff * w).sum() / n, _mean_op),
        "sampler_trainer/logp_diff_max": ((diff * w).max() if diff.numel() else diff.sum(), _max_op),
        "sampler_trainer/mult_prob_error_mean": ((mult_err * w).sum() / n, _mean_op),
        "sampler_trainer/mult_prob_error_max": (mult_err.max() if mult_err.numel() else mult_err.sum(), _max_op),
        "sampler_trainer/prob_diff_mean": (pdiff.sum() / n, _mean_op),
        "sampler_trainer/prob_diff_max": (pdiff.max() if pdiff.numel() else pdiff.sum(), _max_op),
        "sampler_trainer/probs_pearson_corr": (_pearson(pro, ptr, w), _mean_op),
    })
    S = _resolve_num_segments(segment_ids, num_segments)

    def per_seq(vals, weights):
        """(sum of vals*weights, sum of weights) per sequence -> [B, nseq]; and a gather back to tokens."""
        if segment_ids is not None:
            s = segment_sum(vals * weights, segment_ids, S)
            c = segment_sum(weights, segment_ids, S)
            s[:, 0], c[:, 0] = 0, 0
            back = lambda q: q.gather(1, segment_ids.long().clamp(0, S - 1))  # noqa: E731
        else:
            s, c = (vals * weights).sum(-1, keepdim=True), weights.sum(-1, keepdim=True)
            back = lambda q: q.expand(-1, vals.shape[1])  # noqa: E731
        return s, c, back

    comp = completion_mask
    if seq_logprob_error_threshold is not None:
        s, c, back = per_seq(mult_err, w)
        bad_any = per_seq(invalid_scored.float(), torch.ones_like(w))[0] > 0
        seq_err = s / c.clamp(min=1.0)
        active = c > 0
        masked = active & ((seq_err > seq_logprob_error_threshold) | bad_any)
        keep_tok = ~back(masked)
        comp = (completion_mask * keep_tok.to(mask_dtype)).to(mask_dtype)
        cnt = masked.float().sum()
        metrics["sampler_trainer/seq_error_masked_count"] = (cnt, _sum_op)
        metrics["sampler_trainer/seq_error_masked_frac"] = (cnt / active.float().sum().clamp(min=1.0), _mean_op)
    asst = comp > 0
    valid = asst & finite
    w = valid.float()
    log_ratio = torch.where(valid, strn - sro, torch.zeros_like(sro))
    token_ratio = torch.where(valid, torch.exp(log_ratio.clamp(-20.0, 20.0)), torch.zeros_like(sro))
    s, c, back = per_seq(log_ratio, w)
    active_seq = c > 0
    seq_mean_lr = s / c.clamp(min=1.0)
    seq_geo = torch.exp(seq_mean_lr.clamp(-20.0, 20.0))
    na = active_seq.float().sum().clamp(min=1.0)
    metrics["sampler_is/seq_kl_mean"] = ((-(seq_mean_lr) * active_seq).sum() / na, _mean_op)
    metrics["sampler_is/seq_geo_ratio_mean"] = ((seq_geo * active_seq).sum() / na, _mean_op)
    metrics["sampler_is/seq_geo_ratio_max"] = ((seq_geo * active_seq).max(), _max_op)
    weights = None
    if sampler_is is not None or sampler_rs is not None:
        weights = torch.ones_like(sro)
        if sampler_is == "token":
            weights = token_ratio
        elif sampler_is == "sequence":
            weights = back(seq_geo ** c.clamp(min=1.0)) if False else back(torch.exp((s).clamp(-20.0, 20.0)))
        if sampler_is is not None and sampler_is_threshold is not None:
            clipped = (weights > sampler_is_threshold) & valid
            metrics["sampler_is/frac_clipped_at_threshold"] = (clipped.float().sum() / w.sum().clamp(min=1.0), _mean_op)
            weights = weights.clamp(max=sampler_is_threshold)
        if sampler_rs is not None:
            lo = -float("inf") if sampler_rs_min is None else sampler_rs_min
            hi = float("inf") if sampler_rs_max is None else sampler_rs_max
            if sampler_rs == "token":
                keep = (token_ratio >= lo) & (token_ratio <= hi)
            else:
                keep = back((seq_geo >= lo) & (seq_geo <= hi))
            rejected = valid & ~keep
            metrics["sampler_rs/rejected_fraction"] = (rejected.float().sum() / w.sum().clamp(min=1.0), _mean_op)
            weights = weights * keep.float()
        weights = (weights * w).detach()
        wn = w.sum().clamp(min=1.0)
        metrics["sampler_is/weight_mean"] = (weights.sum() / wn, _mean_op)
        metrics["sampler_is/weight_min"] = (torch.where(valid, weights, torch.full_like(weights, float("inf"))).min(), _min_op)
        metrics["sampler_is/weight_max"] = (weights.max(), _max_op)
    return metrics, weights, comp


class RepeatIterable:
    """Repeat every batch of `data` `repeat` times, optionally with a seeded shuffle of each repetition's rows."""

    def __init__(self, data, repeat: int = 1, mini_batch_size: Optional[int] = None, shuffle: bool = False, seed: int = 0):
        self._data, self._repeat, self._mb, self._shuffle, self._seed = list(data), repeat, mini_batch_size, shuffle, seed

    def __iter__(self):
        rng = np.random.default_rng(self._seed)
        for _ in range(self._repeat):
            order = rng.permutation(len(self._data)) if self._shuffle else range(len(self._data))
            for i in order:
                yield self._data[i]
