"""Naming, safetensors round trip (incl. LoRA merge and MoE expert stacking), AutoModel."""
import pytest
import torch

from tunix_b200.lora import LoraProvider, apply_lora_to_model
from tunix_b200.models import naming
from tunix_b200.models.automodel import AutoModel, ModelSource
from tunix_b200.models.config import ModelConfig, get_config
from tunix_b200.models.safetensors_loader import create_model_from_safe_tensors, load_safetensors_into
from tunix_b200.models.safetensors_saver import save_lora_merged_model_as_safetensors
from tunix_b200.models.transformer import create_model


@pytest.mark.parametrize("mid,cid,fam", [
    ("meta-llama/Llama-3.1-8B", "llama3p1_8b", "llama3"), ("Qwen/Qwen3-8B", "qwen3_8b", "qwen3"),
    ("Qwen/Qwen3-30B-A3B", "qwen3_30b_a3b", "qwen3"), ("google/gemma-2-9b-it", "gemma2_9b", "gemma2"),
    ("Qwen/Qwen2.5-7B-Instruct", "qwen2p5_7b", "qwen2"), ("google/gemma-3-1b-it", "gemma3_1b", "gemma3"),
    ("meta-llama/Llama-3.2-1B", "llama3p2_1b", "llama3")])
def test_naming(mid, cid, fam):
    n = naming.resolve(mid)
    assert (n.config_id, n.family) == (cid, fam)


def test_preset_param_counts():
    assert abs(get_config("llama3p1_8b").num_params() / 8.03e9 - 1) < 0.01
    assert abs(get_config("qwen3_8b").num_params() / 8.19e9 - 1) < 0.01
    assert abs(get_config("qwen3_30b_a3b").num_params() / 30.5e9 - 1) < 0.02


SMALL = dict(num_layers=2, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2, head_dim=16, num_kv_heads=1)


@pytest.mark.parametrize("extra", [
    dict(family="llama3"), dict(family="qwen3", qk_norm=True), dict(family="qwen2", qkv_bias=True),
    dict(family="gemma2", post_norms=True, norm_add_one=True, weight_tying=True, activation="gelu"),
    dict(family="qwen3", qk_norm=True, num_experts=4, num_experts_per_tok=2, moe_hidden_dim=24)])
def test_safetensors_round_trip(tmp_path, extra):
    cfg = ModelConfig(**SMALL, **extra)
    m = create_model(cfg, seed=0)
    save_lora_merged_model_as_safetensors(m, str(tmp_path))
    m2 = create_model_from_safe_tensors(str(tmp_path), cfg)
    toks = torch.randint(0, 64, (2, 9))
    a, _ = m(toks)
    b, _ = m2(toks)
    assert torch.allclose(a, b, atol=1e-6)


def test_lora_merge_export_matches_adapter_model(tmp_path):
    cfg = ModelConfig(**SMALL)
    m = create_model(cfg, seed=0)
    apply_lora_to_model(m, LoraProvider(rank=4, alpha=8.0))
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("lora_b"):
                p.normal_(0, 0.05)
    save_lora_merged_model_as_safetensors(m, str(tmp_path))
    merged = create_model_from_safe_tensors(str(tmp_path), cfg)
    toks = torch.randint(0, 64, (2, 9))
    assert torch.allclose(m(toks)[0], merged(toks)[0], atol=1e-5)


def test_automodel_random():
    model, path = AutoModel.from_pretrained("meta-llama/Llama-3.2-1B", model_source=ModelSource.RANDOM,
                                            num_layers=1, vocab_size=128, embed_dim=64, hidden_dim=128, num_heads=2,
                                            head_dim=32, num_kv_heads=1)
    assert path is None and model.config.family == "llama3" and len(model.layers) == 1
