"""RL math against closed forms (NumPy), on CPU."""
import math

import numpy as np
import pytest
import torch

from tunix_b200.rl import algo_core, common
from tunix_b200.rl.algorithm_config import GRPOConfig, PPOConfig, DAPOConfig
from tunix_b200.models.config import ModelConfig
from tunix_b200.models.transformer import create_model


def test_grpo_advantages_closed_form():
    r = np.array([1.0, 2.0, 3.0, 6.0, 0.0, 0.0, 4.0, 4.0], np.float32)
    a = algo_core.compute_advantages(r, 4)
    g0 = r[:4]
    assert np.allclose(a[:4], (g0 - g0.mean()) / (g0.std(ddof=1) + 1e-6), atol=1e-5)
    d = algo_core.compute_drgrpo_advantages(r, 4)
    assert np.allclose(d[:4], g0 - g0.mean())
    loo = algo_core.compute_rloo_advantages(r, 4)
    assert np.isclose(loo[0], 1.0 - (2 + 3 + 6) / 3)
    # a group with fewer than two valid members is zeroed
    v = np.array([1, 0, 0, 0, 1, 1, 1, 1], bool)
    a2 = algo_core.compute_advantages(r, 4, valid_mask=v)
    assert np.all(a2[:4] == 0) and a2[6] != 0 or np.allclose(a2[4:], (r[4:] - 2) / (r[4:].std(ddof=1) + 1e-6), atol=1e-5)


def test_gae_matches_loop():
    torch.manual_seed(0)
    B, T = 3, 7
    r, v = torch.randn(B, T), torch.randn(B, T)
    m = torch.ones(B, T)
    m[1, 5:] = 0
    adv, ret = algo_core.compute_gae_advantages(r, v, m, gamma=0.9, gae_lambda=0.8, whiten=False)
    for b in range(B):
        last, nv = 0.0, 0.0
        for t in range(T - 1, -1, -1):
            if m[b, t] > 0:
                delta = r[b, t] + 0.9 * nv - v[b, t]
                last = delta + 0.9 * 0.8 * last
                nv = v[b, t]
                assert abs(adv[b, t].item() - float(last)) < 1e-5


@pytest.mark.parametrize("mode", ["token-mean", "sequence-mean-token-mean", "sequence-mean-token-scale",
                                  "seq-mean-token-sum", "sequence-mean-token-sum-norm"])
def test_aggregate_loss_matches_eager_crosscheck(mode):
    torch.manual_seed(1)
    L = torch.randn(4, 9)
    m = (torch.rand(4, 9) > 0.3).float()
    m[2] = 0
    a = common.aggregate_loss(L, m, mode)
    ref = common.reduced_loss_agg(L, m, mode)
    assert torch.allclose(a.value(), ref, atol=1e-5)
    # packed: two segments per row must equal the same sequences unpacked
    if mode not in ("sequence-mean-token-scale",):
        seg = torch.tensor([[1] * 4 + [2] * 5] * 4)
        ap = common.aggregate_loss(L, m, mode, segment_ids=seg, num_segments=3, norm=8 if "norm" in mode else None)
        rp = common.reduced_loss_agg(L, m, mode, segment_ids=seg, num_segments=3, norm=8 if "norm" in mode else None)
        assert torch.allclose(ap.value(), rp, atol=1e-5)


def test_kl_modes():
    a, b = torch.tensor([-1.0, -2.0]), torch.tensor([-1.5, -1.0])
    assert torch.allclose(common.compute_kl_divergence(a, b, "kl"), a - b)
    assert torch.allclose(common.compute_kl_divergence(a, b, "mse_kl"), 0.5 * (a - b) ** 2)
    d = b - a
    assert torch.allclose(common.compute_kl_divergence(a, b, "low_var_kl"), torch.exp(d) - d - 1)


def _tiny():
    cfg = ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2,
                                           head_dim=16, num_kv_heads=1)
    return create_model(cfg, seed=0)


def _example(B=4, P=5, C=6, with_old=False, with_ref=False):
    g = torch.Generator().manual_seed(0)
    ex = common.TrainExample(
        prompt_ids=torch.randint(1, 64, (B, P), generator=g), prompt_mask=torch.ones(B, P, dtype=torch.int32),
        completion_ids=torch.randint(1, 64, (B, C), generator=g), completion_mask=torch.ones(B, C, dtype=torch.int32),
        advantages=torch.tensor([1.0, -1.0, 0.5, -0.5]))
    ex.completion_mask[0, 4:] = 0
    return ex


def test_grpo_loss_on_policy_gradient_is_policy_gradient():
    model = _tiny()
    ex = _example()
    cfg = GRPOConfig(num_generations=2, beta=0.0)
    out = algo_core.grpo_loss_fn(model, ex, cfg, pad_id=0, eos_id=63)
    # on-policy: ratio == 1, loss value == -mean over sequences of mean-token advantage
    m = ex.completion_mask.float()
    expected = (-(ex.advantages[:, None] * m).sum(-1) / m.sum(-1)).mean()
    assert torch.allclose(out.loss.value(), expected, atol=1e-5)
    out.loss.value().backward()
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in model.parameters())
    assert abs(float(out.aux["pg_clipfrac"])) < 1e-6


def test_grpo_loss_clipping_and_kl():
    model = _tiny()
    ex = _example()
    with torch.no_grad():
        logp = common.compute_per_token_logps(model, ex.prompt_ids, ex.completion_ids, 0, 63,
                                              completion_mask=ex.completion_mask)
    ex.old_per_token_logps = logp - 1.0          # ratio = e: clipped for positive advantages
    ex.ref_per_token_logps = logp - 0.1
    cfg = GRPOConfig(num_generations=2, beta=0.04, epsilon=0.2, use_rollout_logps=False)
    out = algo_core.grpo_loss_fn(model, ex, cfg, pad_id=0, eos_id=63)
    assert float(out.aux["pg_clipfrac"]) > 0.3
    assert abs(float(out.aux["kl"]) - 0.1) < 1e-4
    gs = GRPOConfig(num_generations=2, beta=0.0, loss_algo="gspo-token", use_rollout_logps=False)
    out2 = algo_core.grpo_loss_fn(model, ex, gs, pad_id=0, eos_id=63)
    assert torch.isfinite(out2.loss.value())
    dual = GRPOConfig(num_generations=2, beta=0.0, epsilon_c=3.0, use_rollout_logps=False)
    out3 = algo_core.grpo_loss_fn(model, ex, dual, pad_id=0, eos_id=63)
    assert "pg_clipfrac_lower" in out3.aux


def test_sampler_trainer_agreement_weights():
    ro = torch.log(torch.tensor([[0.5, 0.25, 0.1]]))
    tr = torch.log(torch.tensor([[0.5, 0.5, 0.05]]))
    mask = torch.ones(1, 3)
    met, w, filt = common.sampler_trainer_agreement(ro, tr, mask, sampler_is="token", sampler_is_threshold=1.5)
    assert torch.allclose(w, torch.tensor([[1.0, 1.5, 0.5]]), atol=1e-5)
    assert abs(float(met["sampler_is/frac_clipped_at_threshold"][0]) - 1 / 3) < 1e-6
    met, w, filt = common.sampler_trainer_agreement(ro, tr, mask, seq_logprob_error_threshold=1.2)
    assert filt.sum() == 0 and float(met["sampler_trainer/seq_error_masked_count"][0]) == 1


def test_config_validation():
    with pytest.raises(ValueError):
        GRPOConfig(num_generations=1)
    with pytest.raises(ValueError):
        GRPOConfig(loss_agg_mode="nope")
    assert DAPOConfig(num_generations=4).epsilon_high == 0.28
    assert PPOConfig().epsilon_low == 0.2


def test_align_routed_experts_pads_like_the_trainer_and_replay_reproduces_the_samplers_routing():
    import numpy as np
    import torch
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.rl import common
    L, k = 2, 2
    r = lambda n, base: (np.arange(n * L * k).reshape(n, L, k) % 5 + base).astype(np.int16)  # noqa: E731
    out = common.align_routed_experts([r(5, 0), r(9, 1)], [2, 4], prompt_width=4, completion_width=3)
    assert out.shape == (2, 7, L, k) and out.dtype == np.int16
    a = r(5, 0)                                   # prompt 3 + completion 2: left pad 1, right pad 1
    assert (out[0, 0] == -1).all() and (out[0, 1:4] == a[:3]).all() and (out[0, 4:6] == a[3:]).all() and (out[0, 6] == -1).all()
    b = r(9, 1)                                   # prompt 5 + completion 4: prompt keeps its tail, completion its head
    assert (out[1, :4] == b[1:5]).all() and (out[1, 4:] == b[5:8]).all()
    assert common.align_routed_experts([r(5, 0), None], [2, 4], 4, 3) is None and common.align_routed_experts(None, [], 4, 3) is None
    # replay: a model forced to the routing that ANOTHER set of router weights chose gives the log-probs of that routing
    cfg = ModelConfig.tiny_llama().replace(num_layers=2, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2, head_dim=16,
                                           num_kv_heads=1, num_experts=4, num_experts_per_tok=2, moe_hidden_dim=32)
    model = create_model(cfg, seed=0)
    toks = torch.randint(3, 64, (2, 7), generator=torch.Generator().manual_seed(1))
    model(toks, skip_lm_head=True)
    own = model.routed_experts_of_last_forward()                       # [2, 7, L, k]
    assert own.shape == (2, 7, 2, 2)
    forced = (own + 1) % 4                                             # a different, valid choice everywhere
    h_own, _ = model(toks, skip_lm_head=True)
    h_forced, _ = model(toks, skip_lm_head=True, routed_experts=forced)
    assert torch.equal(model.routed_experts_of_last_forward(), forced) and not torch.allclose(h_own, h_forced)
    h_unset, _ = model(toks, skip_lm_head=True, routed_experts=torch.full_like(own, -1))
    assert torch.allclose(h_unset, h_own)                               # -1 leaves every token to the model's router
    lp = common.compute_per_token_logps(model, toks[:, :3], toks[:, 3:], 0, 1, routed_experts=forced.numpy())
    lp2 = common.compute_per_token_logps(model, toks[:, :3], toks[:, 3:], 0, 1)
    assert lp.shape == (2, 4) and not torch.allclose(lp, lp2)


def test_per_token_logps_on_packed_rows_equal_the_padded_ones():
    """Two sequences packed into one row (segment ids, restarted positions, no prompt side) give the same completion
    log-probs as the padded [prompt | completion] layout."""
    import numpy as np
    import torch
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.rl import common, utils as rl_utils
    cfg = ModelConfig.tiny_llama().replace(num_layers=2, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2, head_dim=16,
                                           num_kv_heads=1)
    model = create_model(cfg, seed=0)
    g = torch.Generator().manual_seed(2)
    pad = 0
    prompts = torch.tensor([[pad, pad, 5, 6, 7], [9, 10, 11, 12, 13]])
    pmask = (prompts != pad).int()
    comps = torch.tensor([[20, 21, 22, pad], [30, 31, 32, 33]])
    cmask = (comps != pad).int()
    padded = common.compute_per_token_logps(model, prompts, comps, pad, 1, completion_mask=cmask)
    ex = common.TrainExample(prompt_ids=prompts, prompt_mask=pmask, completion_ids=comps, completion_mask=cmask,
                             advantages=torch.tensor([1.0, -1.0]))
    packed = list(rl_utils.pack_sequences([ex], budget=20, pack_size=1, pad_id=pad, device=torch.device("cpu")))
    assert len(packed) == 1 and packed[0].completion_ids.shape == (1, 20) and packed[0].prompt_ids.shape[1] == 0
    pk = packed[0]
    lp = common.compute_per_token_logps(model, pk.prompt_ids, pk.completion_ids, pad, 1, completion_mask=pk.completion_mask,
                                        segment_ids=pk.segment_ids, segment_positions=pk.segment_positions)
    got = lp[0][pk.completion_mask[0] > 0]
    want = torch.cat([padded[0][:3], padded[1]])                    # sequence 0 has three completion tokens, sequence 1 four
    order = pk.completion_ids[0][pk.completion_mask[0] > 0]
    if int(order[0]) == 30:                                         # the packer may place the longer sequence first
        want = torch.cat([padded[1], padded[0][:3]])
    assert torch.allclose(got, want, atol=1e-5), (got, want)
