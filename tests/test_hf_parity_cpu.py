"""Architecture parity with the Hugging Face implementations: same random weights, same tokens, same logits.

A tiny model of each family is built with `transformers`, its weights are written as safetensors, loaded through
this framework's loader into the generic decoder, and the fp32 logits are compared on CPU."""
import json
import os

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _save(model, path):
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    sd = {k: v.detach().clone().contiguous() for k, v in model.state_dict().items()}
    save_file(sd, os.path.join(path, "model.safetensors"))
    json.dump(model.config.to_dict(), open(os.path.join(path, "config.json"), "w"), default=str)


def _ours(cfg, path):
    from tunix_b200.models import safetensors_loader
    from tunix_b200.models.transformer import create_model
    model = create_model(cfg, seed=1)
    safetensors_loader.load_safetensors_into(model, path)
    return model.eval()


CASES = {
    "llama3": lambda t: (t.LlamaForCausalLM(t.LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                                          num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-5,
                                                          rope_theta=500000.0, tie_word_embeddings=False, max_position_embeddings=64)),
                         dict(family="llama3", norm_eps=1e-5, rope_theta=500000.0)),
    "qwen2": lambda t: (t.Qwen2ForCausalLM(t.Qwen2Config(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                                         num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-6,
                                                         rope_theta=1000000.0, tie_word_embeddings=False, max_position_embeddings=64)),
                        dict(family="qwen2", norm_eps=1e-6, rope_theta=1000000.0, qkv_bias=True)),
    "qwen3": lambda t: (t.Qwen3ForCausalLM(t.Qwen3Config(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                                         num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6,
                                                         rope_theta=1000000.0, tie_word_embeddings=False, max_position_embeddings=64)),
                        dict(family="qwen3", norm_eps=1e-6, rope_theta=1000000.0, qk_norm=True)),
    "gemma2": lambda t: (t.Gemma2ForCausalLM(t.Gemma2Config(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                                            num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                                                            rms_norm_eps=1e-6, rope_theta=10000.0, query_pre_attn_scalar=16,
                                                            sliding_window=8, attn_logit_softcapping=50.0,
                                                            final_logit_softcapping=30.0, max_position_embeddings=64,
                                                            attn_implementation="eager")),
                         None),
    "gemma3": lambda t: (t.Gemma3ForCausalLM(t.Gemma3TextConfig(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=6,
                                                                num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                                                                rms_norm_eps=1e-6, rope_theta=1000000.0, rope_local_base_freq=10000.0,
                                                                query_pre_attn_scalar=16, sliding_window=8, sliding_window_pattern=6,
                                                                max_position_embeddings=64, attn_implementation="eager")),
                         None),
}


@pytest.mark.parametrize("family", sorted(CASES))
def test_logits_match_huggingface(family, tmp_path):
    from tunix_b200.models.config import ModelConfig
    torch.manual_seed(0)
    hf, extra = CASES[family](transformers)
    hf = hf.eval().float()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.05)
    _save(hf, str(tmp_path))
    c = hf.config
    if family in ("gemma2", "gemma3"):
        from tunix_b200.models.config import get_config
        cfg = get_config("gemma2_2b" if family == "gemma2" else "gemma3_1b").replace(num_layers=c.num_hidden_layers, vocab_size=128, embed_dim=64, hidden_dim=96, num_heads=4, head_dim=16,
                                              num_kv_heads=2, dtype=torch.float32, max_position=64, sliding_window=8,
                                              query_pre_attn_scalar=16.0)
        ours = _ours(cfg, str(tmp_path))
        toks = torch.randint(0, 128, (2, 17))
        with torch.no_grad():
            want, got = hf(toks).logits.float(), ours(toks)[0].float()
        assert torch.allclose(got, want, atol=5e-4, rtol=2e-3), float((got - want).abs().max())
        return
    cfg = ModelConfig(num_layers=2, vocab_size=128, embed_dim=64, hidden_dim=96, num_heads=4, head_dim=16, num_kv_heads=2,
                      dtype=torch.float32, max_position=64, weight_tying=False, **extra)
    ours = _ours(cfg, str(tmp_path))
    toks = torch.randint(0, 128, (2, 17))
    with torch.no_grad():
        want = hf(toks).logits.float()
        got = ours(toks)[0].float()
    assert got.shape == want.shape
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), float((got - want).abs().max())


GEMMA4_CASES = {
    # per-layer inputs, kv sharing over the last 4 layers, double-wide MLP in the sharing layers
    "ple_shared": dict(hf=dict(num_hidden_layers=8, hidden_size_per_layer_input=8, vocab_size_per_layer_input=128,
                               num_kv_shared_layers=4, use_double_wide_mlp=True, num_key_value_heads=1),
                       ours=dict(num_layers=8, per_layer_input_dim=8, num_kv_shared_layers=4, kv_shared_hidden_dim=192,
                                 num_kv_heads=1, layer_pattern=("local", "local", "local", "global"))),
    # keys double as values on the global layers, fewer global kv heads
    "k_eq_v": dict(hf=dict(num_hidden_layers=4, hidden_size_per_layer_input=0, attention_k_eq_v=True,
                           num_global_key_value_heads=1, num_key_value_heads=2),
                   ours=dict(num_layers=4, k_eq_v_global=True, num_global_kv_heads=1, num_kv_heads=2,
                             layer_pattern=("local", "local", "local", "global"))),
    # MoE block beside the dense MLP
    "moe": dict(hf=dict(num_hidden_layers=4, hidden_size_per_layer_input=0, enable_moe_block=True, num_experts=4,
                        top_k_experts=2, moe_intermediate_size=32, num_key_value_heads=2),
                ours=dict(num_layers=4, num_experts=4, num_experts_per_tok=2, moe_hidden_dim=32, num_kv_heads=2,
                          layer_pattern=("local", "local", "local", "global"))),
}


@pytest.mark.parametrize("case", sorted(GEMMA4_CASES))
def test_gemma4_logits_match_huggingface(case, tmp_path):
    from tunix_b200.models import safetensors_loader
    from tunix_b200.models.gemma4 import Gemma4Config
    from tunix_b200.models.transformer import create_model
    t = transformers
    if not hasattr(t, "Gemma4ForCausalLM"):
        pytest.skip("transformers without Gemma 4")
    spec = GEMMA4_CASES[case]
    torch.manual_seed(0)
    L = spec["hf"]["num_hidden_layers"]
    hcfg = t.Gemma4TextConfig(vocab_size=128, hidden_size=64, intermediate_size=96, num_attention_heads=4, head_dim=16,
                              global_head_dim=32, rms_norm_eps=1e-6, sliding_window=8, max_position_embeddings=64,
                              final_logit_softcapping=30.0, attn_implementation="eager",
                              layer_types=["sliding_attention" if (i + 1) % 4 else "full_attention" for i in range(L)],
                              **spec["hf"])
    hf = t.Gemma4ForCausalLM(hcfg).eval().float()
    for n, p in hf.named_parameters():
        torch.nn.init.normal_(p, std=0.05)
        if "norm" in n or n.endswith("scale"):
            p.data.add_(1.0)
    for n, b in hf.named_buffers():
        if n.endswith("layer_scalar"):
            b.fill_(0.5 + 0.1 * int(n.split(".")[2]))
    _save(hf, str(tmp_path))
    cfg = Gemma4Config._base(vocab_size=128, embed_dim=64, hidden_dim=96, num_heads=4, head_dim=16, global_head_dim=32,
                             sliding_window=8, max_position=64, dtype=torch.float32, **spec["ours"])
    ours = create_model(cfg, seed=1)
    unused = safetensors_loader.load_safetensors_into(ours, str(tmp_path))
    # the only checkpoint tensors without a home are the k/v weights HF keeps for the kv-sharing layers
    assert all(".self_attn.k_" in k or ".self_attn.v_" in k for k in unused), unused
    ours.eval()
    toks = torch.randint(1, 128, (2, 19))
    with torch.no_grad():
        want = hf(toks, use_cache=True).logits.float()
        got = ours(toks)[0].float()
    assert torch.allclose(got, want, atol=5e-4, rtol=2e-3), float((got - want).abs().max())
    # prefill + one decode step through the dense cache (kv-sharing layers read their source layer's cache)
    with torch.no_grad():
        cache = ours.init_cache(2, 32)
        _, cache = ours(toks[:, :18], cache=cache)
        step, _ = ours(toks[:, 18:19], positions=torch.full((2, 1), 18, dtype=torch.int32), cache=cache)
    assert torch.allclose(step[:, 0].float(), want[:, 18], atol=5e-4, rtol=2e-3)
    # gradients reach every parameter
    ours.train()
    loss = ours(toks)[0].float().logsumexp(-1).mean()
    loss.backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in ours.parameters())


def test_gemma4_export_round_trip(tmp_path):
    """Saver -> loader round trip of a Gemma-4 model with every special tensor (per-layer inputs, experts, router,
    layer scalars), and the exported names are the ones `transformers` uses."""
    from tunix_b200.models import safetensors_loader, safetensors_saver
    from tunix_b200.models.gemma4 import Gemma4Config
    from tunix_b200.models.transformer import create_model
    cfg = Gemma4Config._base(vocab_size=64, embed_dim=32, hidden_dim=48, num_layers=4, num_heads=2, num_kv_heads=1, head_dim=16,
                             global_head_dim=32, sliding_window=8, max_position=32, per_layer_input_dim=8, num_experts=4,
                             num_experts_per_tok=2, moe_hidden_dim=16, layer_pattern=("local", "global"), dtype=torch.float32)
    a = create_model(cfg, seed=5)
    with torch.no_grad():
        for i, layer in enumerate(a.layers):
            layer.layer_scalar.fill_(0.5 + i)
    safetensors_saver.save_lora_merged_model_as_safetensors(a, str(tmp_path))
    from safetensors import safe_open
    with safe_open(str(tmp_path / "model.safetensors"), "pt") as f:
        keys = set(f.keys())
    assert {"model.embed_tokens_per_layer.weight", "model.layers.0.experts.gate_up_proj", "model.layers.1.router.proj.weight",
            "model.layers.2.router.per_expert_scale", "model.layers.3.layer_scalar"} <= keys
    b = create_model(cfg, seed=6)
    assert safetensors_loader.load_safetensors_into(b, str(tmp_path)) == []
    toks = torch.randint(1, 64, (2, 9))
    with torch.no_grad():
        assert torch.equal(a(toks)[0], b(toks)[0])


@pytest.mark.parametrize("family", sorted(CASES))
def test_config_from_hf_and_logit_checker(family, tmp_path, capsys):
    """The checkpoint directory alone (config.json + safetensors) is enough: the config is derived from the Hugging
    Face one and the checker reports agreement with the Hugging Face forward pass."""
    from tunix_b200.models import logit_checker
    from tunix_b200.models.hf_config import config_from_hf
    torch.manual_seed(0)
    hf, _ = CASES[family](transformers)
    hf = hf.eval().float()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.05)
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    cfg = config_from_hf(str(tmp_path), dtype=torch.float32)
    assert cfg.family == family and cfg.num_layers == hf.config.num_hidden_layers and cfg.head_dim == 16
    if family == "gemma3":
        assert cfg.layer_pattern == ("local",) * 5 + ("global",) and cfg.local_rope_theta == 10000.0 and cfg.qk_norm
    if family == "gemma2":
        assert cfg.layer_pattern == ("local", "global") and cfg.attn_logit_softcap == 50.0 and cfg.sliding_window == 8
    if family == "qwen2":
        assert cfg.qkv_bias
    rc = logit_checker.main(["--model-path", str(tmp_path), "--tokens", "17", "--atol", "1e-3"])
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and out["ok"] and out["top1_agreement"] == 1.0 and out["kl_ref_to_ours"] < 1e-6, out
    # a wrong architecture is caught, not waved through
    bad = logit_checker.check(str(tmp_path), tokens=17, config_overrides={"norm_eps": 0.5})
    assert bad["max_abs_diff"] > 1e-3


def test_automodel_reads_an_unnamed_checkpoint_directory_and_moe_config(tmp_path):
    from tunix_b200.models.automodel import AutoModel
    from tunix_b200.models.hf_config import config_from_hf
    torch.manual_seed(0)
    hf, _ = CASES["qwen3"](transformers)
    hf = hf.eval().float()
    hf.save_pretrained(str(tmp_path / "my-finetune"), safe_serialization=True)
    model, path = AutoModel.from_pretrained(str(tmp_path / "my-finetune"), dtype=torch.float32)
    toks = torch.randint(0, 128, (1, 9))
    with torch.no_grad():
        assert torch.allclose(model.eval()(toks)[0].float(), hf(toks).logits, atol=2e-4, rtol=1e-3)
    assert path == str(tmp_path / "my-finetune")
    with pytest.raises((KeyError, ValueError)):
        AutoModel.from_pretrained("no-such-model-anywhere")
    moe = config_from_hf({"model_type": "qwen3_moe", "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 4,
                          "head_dim": 128, "num_hidden_layers": 48, "vocab_size": 151936, "intermediate_size": 6144,
                          "moe_intermediate_size": 768, "num_experts": 128, "num_experts_per_tok": 8, "norm_topk_prob": True,
                          "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 40960, "torch_dtype": "bfloat16",
                          "router_aux_loss_coef": 0.001})
    from tunix_b200.models.config import ModelConfig
    want = ModelConfig.qwen3_30b_a3b()
    for f in ("num_layers", "embed_dim", "num_heads", "num_kv_heads", "head_dim", "num_experts", "num_experts_per_tok",
              "moe_hidden_dim", "vocab_size", "qk_norm", "rope_theta", "router_aux_loss_coef"):
        assert getattr(moe, f) == getattr(want, f), f
    assert moe.dtype == torch.bfloat16
    llama = config_from_hf({"model_type": "llama", "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
                            "num_hidden_layers": 32, "vocab_size": 128256, "intermediate_size": 14336, "rms_norm_eps": 1e-5,
                            "rope_theta": 500000.0, "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}})
    assert llama.head_dim == 128 and llama.rope_llama3_scaling["factor"] == 8.0 and llama.family == "llama3"
    with pytest.raises(ValueError, match="model_type"):
        config_from_hf({"model_type": "mamba", "hidden_size": 8, "num_attention_heads": 1, "num_hidden_layers": 1, "vocab_size": 8})
