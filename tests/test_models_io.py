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


def test_reads_a_checkpoint_that_orbax_wrote_in_its_ocdbt_layout():
    """tests/data/orbax_ocdbt_checkpoint is the checkpoint fixture of the reference's own trainer tests (two dense
    layers w1 [2,4] / w2 [4,2], fp32, zstd-compressed zarr chunks inside an OCDBT store)."""
    import os
    import numpy as np
    import torch
    from tunix_b200.sft import ocdbt
    from tunix_b200.sft.checkpoint_manager import CheckpointManager, _load_item
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "orbax_ocdbt_checkpoint")
    store = ocdbt.OcdbtStore(os.path.join(root, "model_params")).items()
    assert len(store) == 17 and "w1.kernel.value/.zarray" in store and "w2.kernel.value/1.0" in store
    tree = ocdbt.load_tree(os.path.join(root, "model_params"))
    assert sorted(tree) == [("w1", "bias", "value"), ("w1", "kernel", "value"), ("w2", "bias", "value"), ("w2", "kernel", "value")]
    k1 = tree[("w1", "kernel", "value")]
    assert k1.shape == (2, 4) and k1.dtype == np.float32 and abs(float(k1[0, 0]) - 0.7567299) < 1e-6
    assert abs(float(k1[1, 3]) - (-0.7722851)) < 1e-6                       # last chunk (1.1) landed in its corner
    assert tree[("w2", "kernel", "value")].shape == (4, 2) and float(np.abs(tree[("w1", "bias", "value")]).sum()) == 0.0
    item = _load_item(os.path.join(root, "model_params"))
    assert torch.equal(item["w1"]["kernel"]["value"], torch.from_numpy(k1))
    assert CheckpointManager(os.path.dirname(root)).all_steps() == []       # the directory name is not a step number

    # restore into a module whose parameter names match the tree ('<layer>.<kernel|bias>.value')
    class Leaf(torch.nn.Module):
        def __init__(self, *shape):
            super().__init__()
            self.value = torch.nn.Parameter(torch.zeros(*shape))

    class Layer(torch.nn.Module):
        def __init__(self, i, o):
            super().__init__()
            self.kernel, self.bias = Leaf(i, o), Leaf(o)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w1, self.w2 = Layer(2, 4), Layer(4, 2)
    import shutil, tempfile
    with tempfile.TemporaryDirectory() as tmp:
        shutil.copytree(root, os.path.join(tmp, "1"))
        net = Net()
        step, meta = CheckpointManager(tmp).maybe_restore(net)
        assert step == 1 and meta == {}
        assert torch.equal(net.w2.kernel.value.detach(), torch.from_numpy(tree[("w2", "kernel", "value")]))


def test_family_modules_give_the_family_class_and_presets():
    import pytest
    from tunix_b200.models.gemma3 import model as gemma3_lib
    from tunix_b200.models.llama3 import model as llama_lib, params as llama_params
    from tunix_b200.models.qwen3 import model as qwen3_lib
    assert {"llama3p1_8b", "llama3p2_1b", "tiny_llama"} <= set(llama_lib.presets()) and "qwen3_8b" in qwen3_lib.presets()
    assert "qwen3_8b" not in llama_lib.presets() and "gemma3_1b" in gemma3_lib.presets()
    m = llama_lib.Llama3(llama_lib.ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2,
                                                                     head_dim=16, num_kv_heads=1))
    import torch
    assert m(torch.randint(0, 64, (1, 5)))[0].shape == (1, 5, 64)
    with pytest.raises(ValueError, match="family"):
        qwen3_lib.Qwen3(llama_lib.ModelConfig.tiny_llama())
    with pytest.raises(ValueError, match="loader serves"):
        llama_params.create_model_from_safe_tensors("/nowhere", qwen3_lib.ModelConfig.qwen3_0p6b())
    assert llama_params.key_mapping(llama_lib.ModelConfig.tiny_llama())
    from tunix_b200.rl.grpo import dapo_learner, drgrpo_learner
    assert dapo_learner.DAPOConfig(num_generations=2).epsilon_high == 0.28 and drgrpo_learner.DrGRPOLearner.__name__ == "DrGRPOLearner"
