"""RL token kernels (clipped objective + KL with analytic derivatives, GAE scan) against PyTorch autograd."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _torch_ref(logp, old, ref, adv, mask, is_w, eps, eps_high, eps_c, kl_mode, kl_clamp):
    from tunix_b200.rl import common
    active = mask > 0
    lr = (torch.where(active, logp, torch.zeros_like(logp)) - torch.where(active, old, torch.zeros_like(old))).clamp(-20, 20)
    ratio = torch.exp(lr)
    a = torch.where(active, adv[:, None].expand_as(ratio), torch.zeros_like(ratio))
    l1, l2 = -a * ratio, -a * ratio.clamp(1 - eps, 1 + eps_high)
    loss = torch.maximum(l1, l2)
    if eps_c is not None:
        loss = torch.where(a < 0, torch.minimum(-eps_c * a, loss), loss)
    if is_w is not None:
        loss = loss * torch.where(active, is_w, torch.zeros_like(is_w))
    kl = common.compute_kl_divergence(logp, ref, kl_mode, kl_clamp)
    return loss, torch.where(active, kl, torch.zeros_like(kl))


@pytest.mark.parametrize("kl_mode,eps_c,use_isw", [("kl", None, False), ("mse_kl", 3.0, True), ("low_var_kl", None, True)])
def test_policy_loss_kernel_matches_autograd(kl_mode, eps_c, use_isw):
    from tunix_b200.rl.algo_core import _PolicyLossFn
    torch.manual_seed(0)
    B, T = 16, 200
    dev = "cuda"
    logp = (-torch.rand(B, T, device=dev) * 3).requires_grad_()
    old = (logp.detach() + torch.randn(B, T, device=dev) * 0.3)
    ref = (logp.detach() + torch.randn(B, T, device=dev) * 0.3)
    adv = torch.randn(B, device=dev)
    mask = (torch.rand(B, T, device=dev) > 0.2).float()
    is_w = torch.rand(B, T, device=dev) + 0.5 if use_isw else None
    gp, gk = torch.randn(B, T, device=dev), torch.randn(B, T, device=dev)
    pg, kl, flags = _PolicyLossFn.apply(logp, old, ref, adv, mask, is_w, 0.2, 0.28, eps_c, kl_mode, 10.0)
    ((pg * gp).sum() + (kl * gk).sum()).backward()
    got = logp.grad.clone()
    logp.grad = None
    rpg, rkl = _torch_ref(logp, old, ref, adv, mask, is_w, 0.2, 0.28, eps_c, kl_mode, 10.0)
    ((rpg * gp).sum() + (rkl * gk).sum()).backward()
    assert torch.allclose(pg, rpg, atol=1e-5, rtol=1e-4) and torch.allclose(kl, rkl, atol=1e-5, rtol=1e-4)
    assert torch.allclose(got, logp.grad, atol=1e-4, rtol=1e-3)
    assert flags.shape == (2, B, T) and float(flags[0].sum()) > 0


def test_gae_scan_matches_cpu_loop():
    from tunix_b200.rl.algo_core import compute_gae_advantages
    torch.manual_seed(1)
    B, T = 9, 300
    r, v = torch.randn(B, T), torch.randn(B, T)
    m = (torch.rand(B, T) > 0.15).float()
    m[:, :3] = 0
    a_cpu, ret_cpu = compute_gae_advantages(r, v, m, 0.99, 0.95, whiten=False)
    a_gpu, ret_gpu = compute_gae_advantages(r.cuda(), v.cuda(), m.cuda(), 0.99, 0.95, whiten=False)
    assert torch.allclose(a_gpu.cpu(), a_cpu, atol=1e-4, rtol=1e-4) and torch.allclose(ret_gpu.cpu(), ret_cpu, atol=1e-4, rtol=1e-4)


def test_agentic_grpo_with_engine_server_mode():
    """Agentic GRPO on the paged engine in server mode: every model call is its own request to the engine's
    server; weights are synchronised between steps with the server paused."""
    from tests.test_sampler_cpu import CharTok
    from tunix_b200 import _lib, optim
    from tunix_b200.common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.rl.agentic.agentic_grpo_learner import AgenticGRPOLearner
    from tunix_b200.rl.agentic.parser.chat_template_parser import get_parser
    from tunix_b200.rl.algorithm_config import GRPOConfig
    from tunix_b200.rl.rl_cluster import RLCluster
    cfg = ModelConfig(family="qwen3", num_layers=2, vocab_size=256, embed_dim=128, hidden_dim=256, num_heads=2, head_dim=64,
                      num_kv_heads=1, qk_norm=True, dtype=torch.bfloat16, max_position=128)
    dev = torch.device("cuda")
    actor, ref = create_model(cfg, device=dev, seed=0), create_model(cfg, device=dev, seed=0)
    tc = RLTrainingConfig(eval_every_n_steps=1000, max_steps=2, actor_optimizer=optim.AdamW(1e-3), mini_batch_size=2,
                          train_micro_batch_size=2)
    rc = RolloutConfig(max_tokens_to_generate=6, max_prompt_length=16, temperature=1.0, seed=1, kv_cache_size=64, eos_tokens=[255])
    cl = RLCluster(actor=actor, reference=ref, tokenizer=CharTok(), cluster_config=ClusterConfig(
        role_to_mesh={}, training_config=tc, rollout_config=rc, rollout_engine="paged"))

    def length_reward(prompts, completions, completion_lengths=None, **kw):
        return [float(n % 3) for n in completion_lengths]
    learner = AgenticGRPOLearner(cl, [length_reward], GRPOConfig(num_generations=2, beta=0.04), max_concurrency=4,
                                 chat_parser=get_parser("raw"), server_mode=True)
    served = []
    orig = learner._server_call

    def counting(ids, mt):
        served.append(len(ids))
        return orig(ids, mt)
    learner._server_call = counting
    learner.train([{"prompts": ["ab", "cd"]}, {"prompts": ["ef", "gh"]}])
    _lib.raise_if_kernel_error()
    assert cl.global_steps == 2 and learner.policy_version == 2
    assert len(served) == 8                  # 2 steps x 2 prompts x 2 generations, one request each


def test_disaggregated_grpo_on_two_gpus_syncs_weights_peer_to_peer(tmp_path):
    """Rank 0 trains, rank 1 samples on the paged engine; after the run the sampler's weights (built from another seed)
    equal the actor's: they crossed NVLink through the reshard plan's block pulls."""
    import json
    import subprocess
    import sys
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "res.json")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29771", os.path.join(root, "tests", "rl_placement_worker.py"), out]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    r = json.load(open(out))
    assert r[0]["controller"] and not r[1]["controller"] and r[0]["steps"] == 2
    assert r[1]["served"] == 2 and r[0]["rounds"] == 2            # one generation round per step; the reference is local
    assert r[0]["fused"] and r[1]["fused"] and r[1]["sync_bytes"] > 0
    assert r[0]["max_abs_diff"] == 0.0
