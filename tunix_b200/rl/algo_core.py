"""RL algorithm math: GAE, whitening, PPO / GRPO (GSPO-token, dual-clip) losses, advantage estimators.

Follows tunix/rl/algo_core.py: GAE scan + masked whitening (:33-162), `ppo_policy_loss_fn` (:170-299),
`ppo_value_loss_fn` (:302-392), `grpo_loss_fn` (:400-763), advantage estimators grpo / grpo-loo / rloo /
drgrpo (:801-994). Everything is fp32 torch on the device of its inputs; estimators run on the host (NumPy)
exactly like the reference.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..sft.utils import LossOutput, WeightedMetric
from . import common, function_registry

MIN_VALID_TRAJECTORIES_FOR_ADVANTAGE = 2


# ------------------------------------------------------------------------- GAE
def masked_mean(x, mask, dim=None):
    m = mask.float()
    return (x * m).sum(dim) / m.sum(dim).clamp(min=1e-8)


def masked_var(x, mask, unbiased: bool = True):
    m = mask.float()
    mean = masked_mean(x, m)
    var = masked_mean((x - mean) ** 2, m)
    n = m.sum()
    if unbiased and n > 1:
        var = var * n / (n - 1)
    return var


def masked_whiten(x, mask, shift_mean: bool = True):
    mean, var = masked_mean(x, mask), masked_var(x, mask)
    out = (x - mean) * torch.rsqrt(var + 1e-8)
    return out if shift_mean else out + mean


def compute_gae_advantages(rewards, values, mask, gamma: float = 1.0, gae_lambda: float = 0.95, whiten: bool = True):
    """Reverse scan: delta_t = r_t + gamma V_{t+1} - V_t; A_t = delta_t + gamma*lambda A_{t+1}.
    Masked steps pass the running state through unchanged. Returns (advantages, returns)."""
    r, v, m = rewards.float(), values.float(), mask.float()
    B, T = r.shape
    if r.is_cuda:
        from ..ops import kernels as K
        adv, returns = K.gae_scan(r, v, m, gamma, gae_lambda)        # one thread per sequence walks T backwards
        if whiten:
            adv = masked_whiten(adv, m)
        return adv * m, returns
    adv = torch.zeros_like(r)
    next_v = torch.zeros(B, device=r.device)
    last = torch.zeros(B, device=r.device)
    for t in range(T - 1, -1, -1):
        delta = r[:, t] + gamma * next_v - v[:, t]
        cur = delta + gamma * gae_lambda * last
        on = m[:, t] > 0
        last = torch.where(on, cur, last)
        next_v = torch.where(on, v[:, t], next_v)
        adv[:, t] = last
    returns = adv + v
    if whiten:
        adv = masked_whiten(adv, m)
    return adv * m, returns


# ------------------------------------------------------------------ PPO losses
@function_registry.register_policy_loss_fn("ppo")
def ppo_policy_loss_fn(model, train_example, algo_config, pad_id, eos_id, **kwargs) -> LossOutput:
    eps_low = getattr(algo_config, "epsilon_low", None) or algo_config.epsilon
    eps_high = getattr(algo_config, "epsilon_high", None) or algo_config.epsilon
    eps_c = getattr(algo_config, "epsilon_c", None)
    entropy_coef = getattr(algo_config, "entropy_coef", None)
    mask = train_example.completion_mask.float()
    logp, ent = common.compute_per_token_logps(
        model, train_example.prompt_ids, train_example.completion_ids, pad_id, eos_id,
        completion_mask=train_example.completion_mask, stop_gradient=False, return_entropy=True,
        temperature=getattr(algo_config, "temperature", None), chunk_size=kwargs.get("compute_logps_chunk_size", 0))
    old = train_example.old_per_token_logps
    old = logp.detach() if old is None else old.float()
    adv = train_example.advantages.float()
    if adv.dim() == 1:
        adv = adv[:, None]
    lr = (logp - old).clamp(-20.0, 20.0)
    ratio = torch.exp(lr)
    l1 = -adv * ratio
    l2 = -adv * ratio.clamp(1.0 - eps_low, 1.0 + eps_high)
    loss = torch.maximum(l1, l2)
    clipfrac = masked_mean((l2 > l1).float(), mask)
    aux = {"pg_clipfrac": clipfrac.detach(), "ppo_kl": masked_mean(-lr.detach(), mask)}
    if eps_c is not None:
        l3 = -eps_c * adv
        dual = torch.minimum(l3, loss)
        aux["pg_clipfrac_lower"] = masked_mean(((loss > l3) & (adv < 0)).float(), mask).detach()
        loss = torch.where(adv < 0, dual, loss)
    mode = getattr(algo_config, "loss_agg_mode", "token-mean")
    pg = common.aggregate_loss(loss, mask, mode)
    total_sum = pg.sum
    if entropy_coef:
        e = common.aggregate_loss(ent, mask, mode)
        total_sum = total_sum - entropy_coef * e.sum
        aux["loss/entropy"] = (e.sum / e.denominator.clamp(min=1.0)).detach()
    aux["pg_loss"] = (pg.sum / pg.denominator.clamp(min=1.0)).detach()
    return LossOutput(WeightedMetric(total_sum, pg.denominator, min_denominator=pg.min_denominator), aux)


@function_registry.register_value_loss_fn("ppo")
def ppo_value_loss_fn(model, train_example, algo_config, pad_id, eos_id, **kwargs) -> LossOutput:
    """Clipped value loss 0.5 * max((v - R)^2, (clip(v, v_old +- eps) - R)^2) on completion positions."""
    clip = getattr(algo_config, "clip_range_value", 0.2)
    mask = train_example.completion_mask.float()
    P = train_example.prompt_ids.shape[1]
    scores = common.compute_score(model, train_example.prompt_ids, train_example.completion_ids, pad_id, eos_id,
                                  stop_gradient=False)
    scores = scores[0] if isinstance(scores, tuple) else scores
    v = scores[:, P - 1:-1].float() if scores.dim() == 2 else scores[:, P - 1:-1, 0].float()
    returns, old_v = train_example.returns.float(), train_example.old_values.float()
    v_clipped = old_v + (v - old_v).clamp(-clip, clip)
    l1, l2 = (v - returns) ** 2, (v_clipped - returns) ** 2
    loss = 0.5 * torch.maximum(l1, l2)
    agg = common.aggregate_loss(loss, mask, "token-mean")
    aux = {"vf_clipfrac": masked_mean((l2 > l1).float(), mask).detach(), "values/mean": masked_mean(v.detach(), mask)}
    return LossOutput(agg, aux)


# ------------------------------------------------------------------- GRPO loss
class _PolicyLossFn(torch.autograd.Function):
    """Token-level clipped objective (+ KL) from `csrc/rl_loss.cu`; backward applies the kernel's derivatives."""

    @staticmethod
    def forward(ctx, logp, old, ref, adv, mask, is_w, eps, eps_high, eps_c, kl_mode, kl_clamp):
        from ..ops import kernels as K
        pg, dpg, kl, dkl, flags = K.policy_loss(logp, old, ref, adv, mask, is_w, eps, eps_high, eps_c, kl_mode, kl_clamp)
        ctx.save_for_backward(dpg, dkl if dkl is not None else dpg)
        ctx.has_kl = kl is not None
        ctx.mark_non_differentiable(flags)
        if kl is None:
            kl = torch.zeros((), device=logp.device)
            ctx.mark_non_differentiable(kl)
        return pg, kl, flags

    @staticmethod
    def backward(ctx, g_pg, g_kl, _g_flags):
        dpg, dkl = ctx.saved_tensors
        g = g_pg * dpg
        if ctx.has_kl and g_kl is not None:
            g = g + g_kl * dkl
        return (g,) + (None,) * 10


@function_registry.register_policy_loss_fn("grpo")
def grpo_loss_fn(model, train_example, algo_config, pad_id, eos_id, **kwargs) -> LossOutput:
    beta, eps = algo_config.beta, algo_config.epsilon
    eps_high = getattr(algo_config, "epsilon_high", None) or eps
    eps_c = getattr(algo_config, "epsilon_c", None)
    loss_algo = getattr(algo_config, "loss_algo", "grpo")
    mode = algo_config.loss_agg_mode
    completion_mask = train_example.completion_mask
    segment_ids = getattr(train_example, "segment_ids", None)
    num_segments = getattr(train_example, "num_segments", None)
    comp_seg = None
    if segment_ids is not None:
        comp_seg = segment_ids[:, train_example.prompt_ids.shape[1]:] if segment_ids.shape[1] != completion_mask.shape[1] \
            else segment_ids
    logp, ent = common.compute_per_token_logps(
        model, train_example.prompt_ids, train_example.completion_ids, pad_id, eos_id,
        completion_mask=completion_mask, stop_gradient=False, return_entropy=True, segment_ids=segment_ids,
        segment_positions=getattr(train_example, "segment_positions", None),
        temperature=getattr(algo_config, "temperature", None), chunk_size=kwargs.get("compute_logps_chunk_size", 0),
        routed_experts=getattr(train_example, "routed_experts", None))
    logp = logp.float()
    adv = train_example.advantages.float()
    is_w = train_example.sampler_is_weights
    sa_metrics: dict = {}
    fuse = (algo_config.use_rollout_logps and train_example.old_per_token_logps is not None and is_w is None
            and not train_example.sampler_agreement_applied)
    if fuse:
        sa_metrics, computed_w, filtered = common.sampler_trainer_agreement(
            train_example.old_per_token_logps.float(), logp.detach(), completion_mask,
            sampler_is=algo_config.sampler_is, sampler_is_threshold=algo_config.sampler_is_threshold,
            sampler_rs=algo_config.sampler_rs, sampler_rs_min=algo_config.sampler_rs_min,
            sampler_rs_max=algo_config.sampler_rs_max,
            seq_logprob_error_threshold=algo_config.seq_logprob_error_threshold, segment_ids=comp_seg,
            num_segments=num_segments)
        if algo_config.seq_logprob_error_threshold is not None:
            completion_mask = filtered
        if computed_w is not None:
            is_w = computed_w
    on_policy = train_example.old_per_token_logps is None or (
        fuse and (algo_config.sampler_is is not None or algo_config.sampler_rs is not None
                  or algo_config.seq_logprob_error_threshold is not None))
    old = logp.detach() if on_policy else train_example.old_per_token_logps.float()
    active = (completion_mask > 0) & torch.isfinite(logp) & torch.isfinite(old)
    maskf = completion_mask.float()
    safe_new = torch.where(active, logp, torch.zeros_like(logp))
    safe_old = torch.where(active, old, torch.zeros_like(old))
    lr = safe_new - safe_old
    token_denom = maskf.sum()
    ppo_kl = (-lr).sum().detach() / token_denom.clamp(min=1.0)
    lr = lr.clamp(-20.0, 20.0)
    if loss_algo == "gspo-token":
        if comp_seg is None:
            s = lr.sum(-1, keepdim=True) / maskf.sum(-1, keepdim=True).clamp(min=1.0)
        else:
            S = common._resolve_num_segments(comp_seg, num_segments)
            ssum = common.segment_sum(lr * maskf, comp_seg, S)
            scnt = common.segment_sum(maskf, comp_seg, S)
            s = (ssum / scnt.clamp(min=1.0)).gather(1, comp_seg.long().clamp(0, S - 1))
        lr = (safe_new - safe_new.detach() + s.detach()).clamp(-10.0, 10.0)
    fused_tokens = logp.is_cuda and loss_algo == "grpo"
    aux = {}
    kl_fused = None
    if fused_tokens:
        # ratio, clipping, dual clip, importance weight and KL in one kernel; gradients come from its derivatives
        loss, kl_fused, flags = _PolicyLossFn.apply(
            logp, None if on_policy else old, train_example.ref_per_token_logps, adv, completion_mask.float(),
            None if is_w is None else is_w.float(), eps, eps_high, eps_c, algo_config.kl_loss_mode, algo_config.kl_clamp_value)
        clipfrac = (flags[0] * maskf).sum() / token_denom.clamp(min=1.0)
        with torch.no_grad():       # diagnostics below want the ratio and both branches of the objective
            ratio = torch.exp(lr.detach())
            if adv.dim() == 1:
                adv = adv[:, None].expand_as(ratio)
            adv = torch.where(active & torch.isfinite(adv), adv, torch.zeros_like(adv))
            l1 = -adv * ratio
            l2 = -adv * ratio.clamp(1.0 - eps, 1.0 + eps_high)
        if eps_c is not None:
            lo = common.aggregate_loss(flags[1], maskf, mode, comp_seg, num_segments)
            aux["pg_clipfrac_lower"] = (lo.sum / lo.denominator.clamp(min=lo.min_denominator or 1e-8)).detach()
        if is_w is not None:
            wts = torch.where(active, is_w.float().detach(), torch.zeros_like(loss))
            aux["sampler_is/weight_mean"] = ((wts * maskf).sum() / token_denom.clamp(min=1.0)).detach()
    else:
        ratio = torch.exp(lr)
        if adv.dim() == 1:
            adv = adv[:, None].expand_as(ratio)
        adv = torch.where(active & torch.isfinite(adv), adv, torch.zeros_like(adv))
        l1 = -adv * ratio
        l2 = -adv * ratio.clamp(1.0 - eps, 1.0 + eps_high)
        loss = torch.maximum(l1, l2)
        clipfrac = ((l2 > l1).float() * maskf).sum() / token_denom.clamp(min=1.0)
        if eps_c is not None:
            l3 = -eps_c * adv
            lower = (loss > l3) & (adv < 0)
            loss = torch.where(adv < 0, torch.minimum(l3, loss), loss)
            lo = common.aggregate_loss(lower.float(), maskf, mode, comp_seg, num_segments)
            aux["pg_clipfrac_lower"] = (lo.sum / lo.denominator.clamp(min=lo.min_denominator or 1e-8)).detach()
        if is_w is not None:
            wts = torch.where(active, is_w.float().detach(), torch.zeros_like(loss))
            loss = loss * wts
            aux["sampler_is/weight_mean"] = ((wts * maskf).sum() / token_denom.clamp(min=1.0)).detach()
    norm = kwargs.get("loss_norm")
    pg = common.aggregate_loss(loss, maskf, mode, comp_seg, num_segments, norm=norm)
    total_sum = pg.sum
    aux["reduced_pg_loss"] = common.reduced_loss_agg(loss, maskf, mode, comp_seg, num_segments, norm=norm)
    aux["unreduced_pg_loss"] = (pg.sum / pg.denominator.clamp(min=pg.min_denominator or 1e-8)).detach()
    if train_example.ref_per_token_logps is not None:
        if kl_fused is not None:
            kl = kl_fused
        else:
            kl = common.compute_kl_divergence(logp, train_example.ref_per_token_logps, algo_config.kl_loss_mode,
                                              algo_config.kl_clamp_value)
            kl = torch.where(active, kl, torch.zeros_like(kl))
        klagg = common.aggregate_loss(kl, maskf, mode, comp_seg, num_segments, norm=norm)
        aux["kl"] = ((kl * maskf).sum() / token_denom.clamp(min=1.0)).detach()
        aux["kl_loss"] = (klagg.sum / klagg.denominator.clamp(min=klagg.min_denominator or 1e-8)).detach()
        if beta != 0.0:
            total_sum = total_sum + beta * klagg.sum
    if ent is not None:
        e = common.aggregate_loss(torch.where(active, ent.float().detach(), torch.zeros_like(loss)), maskf, mode, comp_seg,
                                  num_segments, norm=norm)
        aux["entropy"] = (e.sum / e.denominator.clamp(min=e.min_denominator or 1e-8)).detach()
    act_f = active.float()
    na = act_f.sum().clamp(min=1.0)
    r_det = ratio.detach()
    aux.update({
        "pg_clipfrac": clipfrac.detach(), "ppo_kl": ppo_kl,
        "is_ratio/mean": (r_det * act_f).sum() / na,
        "is_ratio/max": torch.where(active, r_det, torch.full_like(r_det, -float("inf"))).max(),
        "is_ratio/min": torch.where(active, r_det, torch.full_like(r_det, float("inf"))).min(),
        "log_ratio/abs_mean": (lr.detach().abs() * act_f).sum() / na,
        "pg_loss/unclipped_mean": (l1.detach() * act_f).sum() / na,
        "pg_loss/clipped_mean": (l2.detach() * act_f).sum() / na,
        "advantage/abs_mean": (adv.abs() * act_f).sum() / na,
        "advantage/max": adv.max(), "advantage/min": adv.min(),
        "advantage/nonzero_frac": ((adv != 0).float() * act_f).sum() / na,
    })
    aux.update(sa_metrics)
    return LossOutput(WeightedMetric(total_sum, pg.denominator, min_denominator=pg.min_denominator), aux)


# --------------------------------------------------------- advantage estimators
def _groups(rewards: np.ndarray, num_generations: int, valid_mask: Optional[np.ndarray]):
    r = np.asarray(rewards, np.float32).reshape(-1, num_generations)
    v = np.ones_like(r, bool) if valid_mask is None else np.asarray(valid_mask, bool).reshape(-1, num_generations)
    return r, v


def _finish(adv: np.ndarray, v: np.ndarray) -> np.ndarray:
    enough = v.sum(1, keepdims=True) >= MIN_VALID_TRAJECTORIES_FOR_ADVANTAGE
    return np.where(v & enough, adv, 0.0).astype(np.float32).reshape(-1)


@function_registry.register_advantage_estimator("grpo")
def compute_advantages(rewards, num_generations: int, valid_mask=None, **_):
    """(r - mean_g) / (std_g(ddof=1) + 1e-6) within each group of `num_generations`."""
    r, v = _groups(rewards, num_generations, valid_mask)
    n = v.sum(1, keepdims=True).clip(min=1)
    mean = (r * v).sum(1, keepdims=True) / n
    var = (((r - mean) ** 2) * v).sum(1, keepdims=True) / (n - 1).clip(min=1)
    return _finish((r - mean) / (np.sqrt(var) + 1e-6), v)


@function_registry.register_advantage_estimator("drgrpo")
def compute_drgrpo_advantages(rewards, num_generations: int, valid_mask=None, **_):
    r, v = _groups(rewards, num_generations, valid_mask)
    n = v.sum(1, keepdims=True).clip(min=1)
    mean = (r * v).sum(1, keepdims=True) / n
    return _finish(r - mean, v)


@function_registry.register_advantage_estimator("rloo")
def compute_rloo_advantages(rewards, num_generations: int, valid_mask=None, **_):
    """Leave-one-out baseline: r_i - mean_{j != i} r_j."""
    r, v = _groups(rewards, num_generations, valid_mask)
    n = v.sum(1, keepdims=True)
    tot = (r * v).sum(1, keepdims=True)
    base = (tot - r * v) / (n - 1).clip(min=1)
    return _finish(r - base, v)


@function_registry.register_advantage_estimator("grpo-loo")
def compute_grpo_loo_advantages(rewards, num_generations: int, valid_mask=None, **_):
    """Leave-one-out mean and std: (r_i - mean_{-i}) / (std_{-i} + 1e-6)."""
    r, v = _groups(rewards, num_generations, valid_mask)
    n = v.sum(1, keepdims=True)
    tot = (r * v).sum(1, keepdims=True)
    tot2 = ((r ** 2) * v).sum(1, keepdims=True)
    n1 = (n - 1).clip(min=1)
    mean = (tot - r * v) / n1
    var = ((tot2 - (r ** 2) * v) / n1 - mean ** 2).clip(min=0.0)
    var = var * n1 / (n1 - 1).clip(min=1)
    return _finish((r - mean) / (np.sqrt(var) + 1e-6), v)


@function_registry.register_advantage_estimator("gae")
def compute_gae(rewards, values, mask, gamma=1.0, gae_lambda=0.95, **_):
    return compute_gae_advantages(rewards, values, mask, gamma, gae_lambda)
