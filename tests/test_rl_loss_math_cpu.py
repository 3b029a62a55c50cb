"""The policy and value objectives against independent eager restatements, over their options; advantage estimators
with invalid rollouts; id handling; the function registry (test model: tests/rl/common_test.py, tests/rl/algo_core_test.py,
tests/rl/ppo/ppo_helpers_test.py). CPU; values AND parameter gradients are compared."""
import itertools

import numpy as np
import pytest
import torch

from tunix_b200.rl import algo_core, common, function_registry, reward_manager  # noqa: F401 (registers the managers)
from tunix_b200.rl.algorithm_config import DAPOConfig, DrGRPOConfig, GRPOConfig, PPOConfig
from tests.test_rl_math import _tiny

PAD, EOS = 0, 63


def _example(seed=0, B=4, P=5, C=7, old_noise=0.0, ref_noise=0.0, model=None):
    g = torch.Generator().manual_seed(seed)
    ex = common.TrainExample(
        prompt_ids=torch.randint(1, 62, (B, P), generator=g), prompt_mask=torch.ones(B, P, dtype=torch.int32),
        completion_ids=torch.randint(1, 62, (B, C), generator=g), completion_mask=torch.ones(B, C, dtype=torch.int32),
        advantages=torch.randn(B, generator=g))
    ex.completion_mask[0, 4:] = 0
    ex.completion_mask[2, 2:] = 0
    if model is not None and (old_noise or ref_noise):
        with torch.no_grad():
            lp = common.compute_per_token_logps(model, ex.prompt_ids, ex.completion_ids, PAD, EOS, completion_mask=ex.completion_mask)
        if old_noise:
            ex.old_per_token_logps = lp + old_noise * torch.randn(lp.shape, generator=g)
        if ref_noise:
            ex.ref_per_token_logps = lp + ref_noise * torch.randn(lp.shape, generator=g)
    return ex


def _agg(L, m, mode, norm=None):
    """Plain restatement of the aggregation modes on unpacked rows."""
    Lm = L * m
    rows = (m.sum(-1) > 0).float().sum()
    if mode == "token-mean":
        return Lm.sum() / m.sum().clamp(min=1)
    if mode == "sequence-mean-token-mean":
        return (Lm.sum(-1) / m.sum(-1).clamp(min=1)).sum() / rows
    if mode == "sequence-mean-token-scale":
        return (Lm.sum(-1) / (norm or L.shape[-1])).sum() / rows
    if mode == "seq-mean-token-sum":
        return Lm.sum() / rows
    if mode == "sequence-mean-token-sum-norm":
        return Lm.sum() / (norm or L.shape[0])
    raise ValueError(mode)


def _kl(lp, ref, mode):
    d = ref - lp
    return {"kl": lp - ref, "mse_kl": 0.5 * (lp - ref) ** 2, "low_var_kl": torch.exp(d) - d - 1}[mode]


def _grads(model):
    out = torch.cat([p.grad.reshape(-1) if p.grad is not None else torch.zeros(p.numel()) for p in model.parameters()])
    model.zero_grad()
    return out


def _reference_grpo(model, ex, cfg):
    lp = common.compute_per_token_logps(model, ex.prompt_ids, ex.completion_ids, PAD, EOS, completion_mask=ex.completion_mask,
                                        stop_gradient=False).float()
    m = ex.completion_mask.float()
    old = lp.detach() if ex.old_per_token_logps is None else ex.old_per_token_logps
    lr = lp - old
    if cfg.loss_algo == "gspo-token":
        s = (lr * m).sum(-1, keepdim=True) / m.sum(-1, keepdim=True).clamp(min=1)
        lr = lp - lp.detach() + s.detach()
    ratio = torch.exp(lr)
    A = ex.advantages[:, None].expand_as(ratio)
    loss = torch.maximum(-A * ratio, -A * ratio.clamp(1 - cfg.epsilon, 1 + cfg.epsilon_high))
    if cfg.epsilon_c is not None:
        loss = torch.where(A < 0, torch.minimum(-cfg.epsilon_c * A, loss), loss)
    total = _agg(loss, m, cfg.loss_agg_mode)
    if ex.ref_per_token_logps is not None and cfg.beta:
        total = total + cfg.beta * _agg(_kl(lp, ex.ref_per_token_logps, cfg.kl_loss_mode), m, cfg.loss_agg_mode)
    return total


_GRID = [dict(), dict(epsilon=0.1, epsilon_high=0.4), dict(epsilon_c=3.0), dict(loss_algo="gspo-token", epsilon=0.05),
         dict(beta=0.3, kl_loss_mode="kl"), dict(beta=0.3, kl_loss_mode="mse_kl"), dict(beta=0.3, kl_loss_mode="low_var_kl")]
_MODES = ["token-mean", "sequence-mean-token-mean", "sequence-mean-token-scale", "seq-mean-token-sum", "sequence-mean-token-sum-norm"]


@pytest.mark.parametrize("opts,mode", [(o, m) for o in _GRID for m in _MODES[:2]] + [({}, m) for m in _MODES[2:]])
def test_grpo_objective_and_gradients_match_the_restatement(opts, mode):
    model = _tiny()
    ex = _example(old_noise=0.25, ref_noise=0.2, model=model)
    cfg = GRPOConfig(num_generations=2, loss_agg_mode=mode, **{"beta": 0.0, **opts})
    out = algo_core.grpo_loss_fn(model, ex, cfg, pad_id=PAD, eos_id=EOS)
    out.loss.value().backward()
    g = _grads(model)
    ref = _reference_grpo(model, ex, cfg)
    ref.backward()
    g_ref = _grads(model)
    assert torch.allclose(out.loss.value(), ref, atol=1e-5, rtol=1e-5)
    assert g_ref.abs().max() > 0 and torch.allclose(g, g_ref, atol=1e-5, rtol=1e-4)
    assert torch.allclose(out.aux["unreduced_pg_loss"] if not cfg.beta else out.aux["reduced_pg_loss"].to(ref.dtype),
                          out.aux["reduced_pg_loss"].to(ref.dtype), atol=1e-5)      # the logged cross-check agrees
    m = ex.completion_mask.bool()
    assert float(out.aux["is_ratio/max"]) >= float(out.aux["is_ratio/mean"]) >= float(out.aux["is_ratio/min"]) > 0
    if "beta" in opts:
        with torch.no_grad():
            lp = common.compute_per_token_logps(model, ex.prompt_ids, ex.completion_ids, PAD, EOS, completion_mask=ex.completion_mask)
        kl = _kl(lp, ex.ref_per_token_logps, cfg.kl_loss_mode)
        assert torch.allclose(out.aux["kl"], kl[m].mean(), atol=1e-5)


def test_clip_fraction_counts_tokens_where_the_clipped_branch_is_active():
    model = _tiny()
    ex = _example(old_noise=0.6, model=model)
    cfg = GRPOConfig(num_generations=2, beta=0.0, epsilon=0.1, loss_agg_mode="token-mean")
    out = algo_core.grpo_loss_fn(model, ex, cfg, pad_id=PAD, eos_id=EOS)
    with torch.no_grad():
        lp = common.compute_per_token_logps(model, ex.prompt_ids, ex.completion_ids, PAD, EOS, completion_mask=ex.completion_mask)
    ratio = torch.exp(lp - ex.old_per_token_logps)
    A = ex.advantages[:, None].expand_as(ratio)
    clipped = ((A > 0) & (ratio > 1.1)) | ((A < 0) & (ratio < 0.9))
    m = ex.completion_mask.bool()
    assert 0 < float(out.aux["pg_clipfrac"]) < 1
    assert torch.allclose(out.aux["pg_clipfrac"], clipped[m].float().mean(), atol=1e-6)
    assert torch.allclose(out.aux["ppo_kl"], (ex.old_per_token_logps - lp)[m].mean(), atol=1e-5)


def test_variant_configs_set_the_documented_defaults():
    d = DAPOConfig(num_generations=2)
    assert (d.beta, d.epsilon_high, d.loss_agg_mode, d.epsilon) == (0.0, 0.28, "token-mean", 0.2)
    r = DrGRPOConfig(num_generations=2)
    assert (r.advantage_estimator, r.loss_agg_mode) == ("drgrpo", "sequence-mean-token-scale")
    assert GRPOConfig(num_generations=2, epsilon=0.3).epsilon_high == 0.3
    for bad in (dict(num_generations=1), dict(loss_algo="x"), dict(loss_agg_mode="x"), dict(kl_loss_mode="x"), dict(epsilon_c=0.5),
                dict(advantage_estimator="nope"), dict(sampler_is="x"), dict(sampler_rs="token")):
        with pytest.raises(ValueError):
            GRPOConfig(**{"num_generations": 2, **bad})
    with pytest.raises(ValueError):
        PPOConfig(epsilon_c=1.0)


@pytest.mark.parametrize("opts", [dict(), dict(epsilon_low=0.1, epsilon_high=0.3), dict(epsilon_c=2.5), dict(entropy_coef=0.05),
                                  dict(loss_agg_mode="sequence-mean-token-mean", entropy_coef=0.01)])
def test_ppo_policy_objective_matches_the_restatement(opts):
    model = _tiny()
    ex = _example(old_noise=0.3, model=model)
    g = torch.Generator().manual_seed(5)
    ex.advantages = torch.randn(ex.completion_ids.shape, generator=g)               # per-token advantages
    cfg = PPOConfig(**opts)
    out = algo_core.ppo_policy_loss_fn(model, ex, cfg, PAD, EOS)
    out.loss.value().backward()
    grads = _grads(model)
    lp, ent = common.compute_per_token_logps(model, ex.prompt_ids, ex.completion_ids, PAD, EOS, completion_mask=ex.completion_mask,
                                             stop_gradient=False, return_entropy=True)
    m = ex.completion_mask.float()
    ratio = torch.exp(lp - ex.old_per_token_logps)
    A = ex.advantages
    loss = torch.maximum(-A * ratio, -A * ratio.clamp(1 - cfg.epsilon_low, 1 + cfg.epsilon_high))
    if cfg.epsilon_c is not None:
        loss = torch.where(A < 0, torch.minimum(-cfg.epsilon_c * A, loss), loss)
    ref = _agg(loss, m, cfg.loss_agg_mode)
    if cfg.entropy_coef:
        ref = ref - cfg.entropy_coef * _agg(ent, m, cfg.loss_agg_mode)
    ref.backward()
    assert torch.allclose(out.loss.value(), ref, atol=1e-5, rtol=1e-5) and torch.allclose(grads, _grads(model), atol=1e-5, rtol=1e-4)
    if cfg.entropy_coef:
        assert float(out.aux["loss/entropy"]) > 0


def test_ppo_value_objective_clips_around_the_old_values():
    from tunix_b200.rl import utils as rl_utils
    critic = rl_utils.create_critic_model(_tiny())
    ex = _example()
    P = ex.prompt_ids.shape[1]
    with torch.no_grad():
        scores = common.compute_score(critic, ex.prompt_ids, ex.completion_ids, PAD, EOS)
        scores = scores[0] if isinstance(scores, tuple) else scores
        v = scores[:, P - 1:-1].float() if scores.dim() == 2 else scores[:, P - 1:-1, 0].float()
    g = torch.Generator().manual_seed(2)
    ex.old_values = v + 0.5 * torch.randn(v.shape, generator=g)
    ex.returns = v + torch.randn(v.shape, generator=g)
    cfg = PPOConfig(clip_range_value=0.2)
    out = algo_core.ppo_value_loss_fn(critic, ex, cfg, PAD, EOS)
    m = ex.completion_mask.float()
    vc = ex.old_values + (v - ex.old_values).clamp(-0.2, 0.2)
    ref = (0.5 * torch.maximum((v - ex.returns) ** 2, (vc - ex.returns) ** 2) * m).sum() / m.sum()
    assert torch.allclose(out.loss.value(), ref, atol=1e-5)
    assert 0 < float(out.aux["vf_clipfrac"]) < 1


@pytest.mark.parametrize("name", ["grpo", "drgrpo", "rloo", "grpo-loo"])
def test_group_estimators_with_invalid_rollouts(name):
    fn = function_registry.get_advantage_estimator(name)
    rng = np.random.default_rng(0)
    r = rng.normal(size=12).astype(np.float32)
    valid = np.ones(12, bool); valid[1] = False; valid[4:7] = False                 # group 1 keeps one valid rollout
    a = fn(r, 4, valid_mask=valid)
    assert a.shape == (12,) and np.all(a[~valid] == 0) and np.all(a[4:8] == 0)       # too few valid: whole group is zero
    g0 = r[[0, 2, 3]]
    if name == "grpo":
        exp = (g0 - g0.mean()) / (g0.std(ddof=1) + 1e-6)
    elif name == "drgrpo":
        exp = g0 - g0.mean()
    elif name == "rloo":
        exp = np.asarray([g0[i] - np.delete(g0, i).mean() for i in range(3)])
    else:
        exp = np.asarray([(g0[i] - np.delete(g0, i).mean()) / (np.delete(g0, i).std(ddof=1) + 1e-6) for i in range(3)])
    np.testing.assert_allclose(a[[0, 2, 3]], exp, rtol=1e-4, atol=1e-5)
    full = fn(r, 4)
    if name in ("grpo", "drgrpo"):
        np.testing.assert_allclose(full.reshape(3, 4).sum(1), 0, atol=1e-4)          # centred within each group
    const = fn(np.ones(4, np.float32), 4)
    assert np.all(np.isfinite(const)) and np.allclose(const, 0)                      # equal rewards: no signal, no NaN


def test_registry_lists_and_rejects_unknown_names():
    assert {"grpo", "ppo"} <= set(function_registry.list_policy_loss_fns()) and "ppo" in function_registry.list_value_loss_fns()
    assert {"grpo", "drgrpo", "rloo", "grpo-loo", "gae"} <= set(function_registry.list_advantage_estimators())
    assert {"sequence-level", "agentic-sequence-level"} <= set(function_registry.list_reward_managers())
    with pytest.raises((KeyError, ValueError)):
        function_registry.get_policy_loss_fn("nope")

    @function_registry.register_advantage_estimator("test-centered")
    def centered(rewards, num_generations, **_):
        r = np.asarray(rewards, np.float32).reshape(-1, num_generations)
        return (r - r.mean(1, keepdims=True)).reshape(-1)
    assert GRPOConfig(num_generations=2, advantage_estimator="test-centered").advantage_estimator == "test-centered"
    np.testing.assert_allclose(function_registry.get_advantage_estimator("test-centered")([1, 3], 2), [-1, 1])


def test_id_handling_helpers():
    ids = torch.tensor([[5, 6, EOS, 7, EOS], [5, 6, 7, 8, 9], [EOS, 1, 2, 3, 4], [5, 62, 6, EOS, 1]])
    assert common.make_completion_mask(ids, EOS).tolist() == [[1, 1, 1, 0, 0], [1, 1, 1, 1, 1], [1, 0, 0, 0, 0], [1, 1, 1, 1, 0]]
    assert common.make_completion_mask(ids, [EOS, 62]).tolist()[3] == [1, 1, 0, 0, 0]               # several stop tokens
    x = torch.tensor([[1, 2, 3]])
    assert common.pad_to_length(x, 5, 9).tolist() == [[1, 2, 3, 9, 9]] and common.pad_to_length(x, 5, 9, left=True).tolist() == [[9, 9, 1, 2, 3]]
    assert common.pad_to_length(x, 2) is x
    assert common.build_positions_from_mask(torch.tensor([[0, 0, 1, 1, 1], [1, 1, 0, 1, 0]])).tolist() == [[0, 0, 0, 1, 2], [0, 1, 1, 2, 2]]
    prompt = torch.tensor([[PAD, PAD, 4, 5]])
    comp = torch.tensor([[6, EOS, 7, PAD]])
    tok, mask, pos = common.process_ids(prompt, comp, PAD, EOS)
    assert tok.tolist() == [[PAD, PAD, 4, 5, 6, EOS, 7, PAD]] and mask.tolist() == [[0, 0, 1, 1, 1, 1, 0, 0]]
    assert pos.tolist() == [[0, 0, 0, 1, 2, 3, 3, 3]]
    assert common.segment_sum(torch.tensor([[1., 2., 3., 4.]]), torch.tensor([[0, 1, 1, 2]]), 3).tolist() == [[1., 5., 4.]]
    logits = torch.randn(2, 3, 11)
    idx = torch.randint(0, 11, (2, 3))
    assert torch.allclose(common.selective_log_softmax(logits, idx), torch.log_softmax(logits, -1).gather(-1, idx[..., None])[..., 0], atol=1e-6)
