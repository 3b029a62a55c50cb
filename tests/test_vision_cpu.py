"""Vision tower, soft-token splice and bidirectional image spans (CPU, tiny sizes)."""
import pytest
import torch

from tunix_b200.models import vision as V
from tunix_b200.testing.common import ToyTransformer


def test_tower_shapes_and_pooling():
    cfg = V.VisionConfig.tiny()
    tower = V.VisionTower(cfg)
    imgs = torch.randn(2, 3, 32, 32, 3)
    out = tower(imgs)
    assert out.shape == (2, 3, 4, 64)
    p = tower.patchify(torch.arange(32 * 32 * 3, dtype=torch.float32).view(1, 32, 32, 3))
    assert p.shape == (1, 16, 8 * 8 * 3) and p[0, 1, 0] == 8 * 3          # second patch starts 8 pixels to the right


def test_merge_places_soft_tokens_in_order():
    text = torch.zeros(2, 6, 3)
    vis = torch.arange(2 * 1 * 2 * 3, dtype=torch.float32).view(2, 1, 2, 3) + 1
    mask = torch.tensor([[0, 1, 1, 0, 0, 0], [0, 0, 0, 0, 0, 0]], dtype=torch.bool)
    out = V.merge_embeddings(text, vis, mask)
    assert torch.equal(out[0, 1], vis[0, 0, 0]) and torch.equal(out[0, 2], vis[0, 0, 1]) and float(out[1].abs().sum()) == 0
    spans = V.image_span_ids(torch.tensor([[5, 9, 9, 9, 9, 7]]), 9, 2)
    assert spans.tolist() == [[0, 1, 1, 2, 2, 0]]


def test_multimodal_forward_backward_and_bidirectional_mask():
    lm = ToyTransformer(vocab_size=128, num_layers=1)
    vc = V.VisionConfig.tiny(image_token_id=100)
    mm = V.Gemma3Multimodal(lm, vc)
    toks = torch.tensor([[1, 100, 100, 100, 100, 7, 8, 9]])
    imgs = torch.randn(1, 1, 32, 32, 3)
    logits, _ = mm(toks, images=imgs)
    assert logits.shape == (1, 8, 128)
    logits.float().logsumexp(-1).sum().backward()
    assert mm.vision_tower.patch_embed.weight.grad is not None and mm.projector.proj.grad.abs().sum() > 0
    # the first image token sees the later ones (bidirectional span): changing the image changes position 1's output
    with torch.no_grad():
        a = mm(toks, images=imgs)[0]
        imgs2 = imgs.clone()
        imgs2[0, 0, 16:, 16:] += 1.0                   # only the last patch row/col -> only the last soft tokens differ
        b = mm(toks, images=imgs2)[0]
    assert not torch.allclose(a[0, 1], b[0, 1])
    text_only = mm(toks[:, 5:])[0]
    assert text_only.shape == (1, 3, 128)


@pytest.mark.parametrize("clipped,standardize", [(False, False), (True, True)])
def test_gemma4_vision_tower_matches_huggingface(clipped, standardize):
    t = pytest.importorskip("transformers")
    if not hasattr(t, "Gemma4VisionConfig"):
        pytest.skip("transformers without Gemma 4")
    from transformers.models.gemma4.modeling_gemma4 import Gemma4VisionModel
    from tunix_b200.models.gemma4_vision import Gemma4VisionConfig, Gemma4VisionTower
    torch.manual_seed(0)
    hcfg = t.Gemma4VisionConfig(hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                                num_key_value_heads=4, head_dim=16, patch_size=4, position_embedding_size=32,
                                pooling_kernel_size=2, use_clipped_linears=clipped, standardize=standardize,
                                attn_implementation="eager")
    hf = Gemma4VisionModel(hcfg).eval().float()
    for n, p in hf.named_parameters():
        torch.nn.init.normal_(p, std=0.1)
        if "norm" in n:
            p.data.add_(1.0)
    for n, b in hf.named_buffers():
        if n.endswith("_min"):
            b.fill_(-1.5)
        elif n.endswith("_max"):
            b.fill_(1.5)
        elif n.endswith("std_bias"):
            b.copy_(torch.randn_like(b) * 0.1)
        elif n.endswith("std_scale"):
            b.copy_(1.0 + torch.rand_like(b))
    ours = Gemma4VisionTower(Gemma4VisionConfig(hidden_size=64, intermediate_size=96, num_layers=2, num_heads=4, num_kv_heads=4,
                                                head_dim=16, patch_size=4, position_embedding_size=32, pooling_kernel_size=2,
                                                use_clipped_linears=clipped, standardize=standardize, dtype=torch.float32))
    missing, unexpected = ours.load_state_dict({k: v for k, v in hf.state_dict().items() if "rotary" not in k}, strict=False)
    assert not unexpected and all("_unit" in m for m in missing), (missing, unexpected)
    # image 0: 6 x 4 patches; image 1: 4 x 4 patches and 8 padding entries
    P = 24
    pos = torch.full((2, P, 2), -1, dtype=torch.long)
    pos[0] = torch.tensor([[x, y] for y in range(4) for x in range(6)])
    pos[1, :16] = torch.tensor([[x, y] for y in range(4) for x in range(4)])
    pix = torch.rand(2, P, 48)
    pix[1, 16:] = 0
    with torch.no_grad():
        want = hf(pix, pos).last_hidden_state
        soft, valid = ours(pix, pos)
    assert valid.sum().item() == 6 + 4 and want.shape[0] == 10
    assert torch.allclose(soft[valid], want, atol=2e-4, rtol=2e-3), float((soft[valid] - want).abs().max())


def test_gemma4_multimodal_matches_huggingface(tmp_path):
    t = pytest.importorskip("transformers")
    if not hasattr(t, "Gemma4VisionConfig"):
        pytest.skip("transformers without Gemma 4")
    from safetensors.torch import save_file
    from transformers.models.gemma4.modeling_gemma4 import Gemma4Model
    from tunix_b200.models import safetensors_loader
    from tunix_b200.models.gemma4 import Gemma4Config
    from tunix_b200.models.gemma4_vision import Gemma4Multimodal, Gemma4VisionConfig
    from tunix_b200.models.transformer import create_model
    torch.manual_seed(0)
    IMG = 120
    tcfg = t.Gemma4TextConfig(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=4, num_attention_heads=4,
                              num_key_value_heads=2, head_dim=16, global_head_dim=32, rms_norm_eps=1e-6, sliding_window=8,
                              max_position_embeddings=64, hidden_size_per_layer_input=8, vocab_size_per_layer_input=128,
                              layer_types=["sliding_attention"] * 3 + ["full_attention"], attn_implementation="eager")
    vcfg = t.Gemma4VisionConfig(hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=2,
                                num_key_value_heads=2, head_dim=16, patch_size=4, position_embedding_size=32,
                                pooling_kernel_size=2, attn_implementation="eager")
    hf = Gemma4Model(t.Gemma4Config(text_config=tcfg, vision_config=vcfg, audio_config=None, image_token_id=IMG)).eval().float()
    for n, p in hf.named_parameters():
        torch.nn.init.normal_(p, std=0.08)
        if "norm" in n:
            p.data.add_(1.0)
    sd = hf.state_dict()
    # key names of a Gemma4ForConditionalGeneration checkpoint: model.language_model.*
    save_file({"model." + k: v.clone().contiguous() for k, v in sd.items() if k.startswith("language_model.")
               and "rotary" not in k}, str(tmp_path / "model.safetensors"))
    lm = create_model(Gemma4Config._base(vocab_size=128, embed_dim=64, hidden_dim=96, num_layers=4, num_heads=4, num_kv_heads=2,
                                         head_dim=16, global_head_dim=32, sliding_window=8, max_position=64,
                                         per_layer_input_dim=8, layer_pattern=("local", "local", "local", "global"),
                                         dtype=torch.float32), seed=3)
    safetensors_loader.load_safetensors_into(lm, str(tmp_path))
    ours = Gemma4Multimodal(lm, Gemma4VisionConfig(hidden_size=32, intermediate_size=48, num_layers=1, num_heads=2, num_kv_heads=2,
                                                   head_dim=16, patch_size=4, position_embedding_size=32, pooling_kernel_size=2,
                                                   image_token_id=IMG, dtype=torch.float32),
                            pad_token_id=tcfg.pad_token_id).eval()
    ours.vision_tower.load_state_dict({k[len("vision_tower."):]: v for k, v in sd.items()
                                       if k.startswith("vision_tower.") and "rotary" not in k}, strict=False)
    ours.embed_vision.load_state_dict({k[len("embed_vision."):]: v for k, v in sd.items() if k.startswith("embed_vision.")},
                                      strict=False)
    P = 24
    pos = torch.full((2, P, 2), -1, dtype=torch.long)
    pos[0] = torch.tensor([[x, y] for y in range(4) for x in range(6)])
    pos[1, :16] = torch.tensor([[x, y] for y in range(4) for x in range(4)])
    pix = torch.rand(2, P, 48)
    toks = torch.randint(1, 100, (2, 20))
    toks[0, 3:9] = IMG          # 6 soft tokens
    toks[1, 5:9] = IMG          # 4 soft tokens
    with torch.no_grad():
        want = hf(input_ids=toks, pixel_values=pix, image_position_ids=pos, use_cache=True).last_hidden_state
        got = ours(toks, pixel_values=pix, pixel_position_ids=pos, skip_lm_head=True)[0]
    assert torch.allclose(got, want, atol=5e-4, rtol=2e-3), float((got - want).abs().max())


def test_gemma4_audio_tower_matches_huggingface():
    t = pytest.importorskip("transformers")
    if not hasattr(t, "Gemma4AudioConfig"):
        pytest.skip("transformers without Gemma 4")
    from transformers.models.gemma4.modeling_gemma4 import Gemma4AudioModel
    from tunix_b200.models.gemma4_audio import Gemma4AudioConfig, Gemma4AudioTower
    torch.manual_seed(0)
    # "sdpa" makes the reference build boolean masks; with "eager" it builds additive ones, which its local attention
    # (written for booleans) reads the wrong way round
    hcfg = t.Gemma4AudioConfig(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, subsampling_conv_channels=[16, 8],
                               conv_kernel_size=5, attention_chunk_size=4, attention_context_left=13, attention_context_right=0,
                               output_proj_dims=24, use_clipped_linears=True, attn_implementation="sdpa")
    hf = Gemma4AudioModel(hcfg).eval().float()
    for n, p in hf.named_parameters():
        torch.nn.init.normal_(p, std=0.15)
        if "norm" in n:
            p.data.add_(1.0)
    for n, b in hf.named_buffers():
        if n.endswith("_min"):
            b.fill_(-2.0)
        elif n.endswith("_max"):
            b.fill_(2.0)
    ours = Gemma4AudioTower(Gemma4AudioConfig(hidden_size=32, num_layers=2, num_heads=4, subsampling_conv_channels=(16, 8),
                                              conv_kernel_size=5, attention_chunk_size=4, output_proj_dims=24,
                                              use_clipped_linears=True, dtype=torch.float32))
    missing, unexpected = ours.load_state_dict({k: v for k, v in hf.state_dict().items()
                                                if "rel_pos_enc" not in k and not k.endswith("softcap")}, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    feats = torch.randn(2, 40, 16)
    mask = torch.ones(2, 40, dtype=torch.bool)
    mask[1, 28:] = False
    with torch.no_grad():
        out = hf(feats, mask)
        got, valid = ours(feats, mask)
    assert torch.equal(valid, out.attention_mask.bool())
    want = out.last_hidden_state
    assert torch.allclose(got[valid], want[valid], atol=3e-4, rtol=2e-3), float((got[valid] - want[valid]).abs().max())


def test_gemma4_image_processing_feeds_the_vision_tower():
    """Aspect-ratio-preserving resize to a patch budget, patch grid positions, padding, placeholder expansion; the
    processed batch goes through the Gemma-4 multimodal model and the number of soft tokens matches the slots."""
    import numpy as np
    from tunix_b200.models.gemma4 import Gemma4Config
    from tunix_b200.models.gemma4_vision import Gemma4Multimodal, Gemma4VisionConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.processors import image_processor as IP
    assert IP.get_target_dimensions(480, 640, 16, 10080, 3) == (1344, 1824)          # 84 x 114 = 9576 patches <= 10080
    assert IP.get_target_dimensions(10, 4000, 16, 90, 3) == (48, 480)                 # the short side keeps one cell
    assert IP.get_target_dimensions(0, 0, 16, 90, 3) == (48, 48)
    p, xy = IP.patchify(np.arange(8 * 12 * 3, dtype=np.float32).reshape(8, 12, 3), 4)
    assert p.shape == (6, 48) and xy.tolist() == [[0, 0], [1, 0], [2, 0], [0, 1], [1, 1], [2, 1]]
    assert p[4, :3].tolist() == [4 * 12 * 3 + 4 * 3, 4 * 12 * 3 + 4 * 3 + 1, 4 * 12 * 3 + 4 * 3 + 2]   # patch (x=1, y=1) starts at pixel (4, 4)
    IMG = 120
    rng = np.random.default_rng(0)
    wide = (rng.random((40, 90, 3)) * 255).astype(np.uint8)
    tall = (rng.random((70, 30)) * 255).astype(np.uint8)                                 # grey-scale input
    toks = [np.asarray([2, 5, IMG, 6, IMG, 7]), np.asarray([2, IMG, 9])]
    vis, out = IP.process_gemma4_inputs([[wide, tall], [tall]], toks, patch_size=4, max_soft_tokens=16, pooling_kernel_size=2,
                                        placeholder_token=IMG, start_token=121, end_token=122, double_new_line_token=123)
    assert vis.patches.shape == (4, 64, 48) and vis.images_per_row == 2 and len(vis.soft_token_counts) == 2
    assert (vis.positions_xy[3] == -1).all() and float(np.abs(vis.patches[3]).sum()) == 0.0      # the missing image of row 1
    for cnt, row in zip(vis.soft_token_counts, out):
        assert int((row == IMG).sum()) == sum(cnt) and int((row == 121).sum()) == len(cnt)
    real = (vis.positions_xy[..., 0] >= 0).sum(1)
    assert [int(r) // 4 for r in real[:3]] == list(vis.soft_token_counts[0]) + list(vis.soft_token_counts[1])
    lm = create_model(Gemma4Config._base(vocab_size=128, embed_dim=64, hidden_dim=96, num_layers=2, num_heads=2, num_kv_heads=1,
                                         head_dim=16, global_head_dim=32, sliding_window=8, max_position=128,
                                         layer_pattern=("local", "global"), dtype=torch.float32), seed=0)
    mm = Gemma4Multimodal(lm, Gemma4VisionConfig(hidden_size=32, intermediate_size=48, num_layers=1, num_heads=2, num_kv_heads=2,
                                                 head_dim=16, patch_size=4, position_embedding_size=64, pooling_kernel_size=2,
                                                 image_token_id=IMG, dtype=torch.float32))
    mm.init_encoder_weights(seed=1, std=0.05)
    width = max(len(r) for r in out)
    batch = torch.as_tensor(np.stack([np.pad(r, (0, width - len(r))) for r in out]))
    with torch.no_grad():
        logits, _ = mm(batch, pixel_values=torch.as_tensor(vis.patches), pixel_position_ids=torch.as_tensor(vis.positions_xy))
    assert logits.shape == (2, width, 128) and torch.isfinite(logits).all()


def test_sampler_prefills_a_multimodal_prompt():
    """The dense Sampler passes image inputs to the prefill of a Gemma-4 multimodal model: the first sampled token
    equals the argmax of a direct forward pass, and changing the image changes the continuation's log-probs."""
    import numpy as np
    from tests.test_sampler_cpu import CharTok
    from tunix_b200.common.configs import CacheConfig
    from tunix_b200.generate.sampler import Sampler
    from tunix_b200.models.gemma4 import Gemma4Config
    from tunix_b200.models.gemma4_vision import Gemma4Multimodal, Gemma4VisionConfig
    from tunix_b200.models.transformer import create_model
    IMG = 120
    lm = create_model(Gemma4Config._base(vocab_size=128, embed_dim=64, hidden_dim=96, num_layers=4, num_heads=2, num_kv_heads=1,
                                         head_dim=16, global_head_dim=32, sliding_window=8, max_position=128, per_layer_input_dim=8,
                                         num_kv_shared_layers=2, layer_pattern=("local", "global"), dtype=torch.float32), seed=0)
    mm = Gemma4Multimodal(lm, Gemma4VisionConfig(hidden_size=32, intermediate_size=48, num_layers=1, num_heads=2, num_kv_heads=2,
                                                 head_dim=16, patch_size=4, position_embedding_size=64, pooling_kernel_size=2,
                                                 image_token_id=IMG, dtype=torch.float32)).init_encoder_weights(seed=2, std=0.2).eval()
    pos = torch.tensor([[x, y] for y in range(4) for x in range(4)])[None]              # 16 patches -> 4 soft tokens
    pix = torch.rand(1, 16, 48, generator=torch.Generator().manual_seed(0))
    prompt = [1, 7, 8] + [IMG] * 4 + [9, 10]
    toks = torch.tensor([prompt])
    with torch.no_grad():
        want = int(mm(toks, pixel_values=pix, pixel_position_ids=pos)[0][0, -1].argmax())
    sampler = Sampler(mm, CharTok(), CacheConfig(64, 4, 1, 16))
    out = sampler(prompt_token_ids=[prompt], max_generation_steps=5, max_prompt_length=len(prompt), return_logprobs=True, eos_tokens=[127],
                  model_inputs={"pixel_values": pix, "pixel_position_ids": pos})
    assert int(out.tokens[0][0]) == want and len(out.tokens[0]) == 5
    other = sampler(prompt_token_ids=[prompt], max_generation_steps=5, max_prompt_length=len(prompt), return_logprobs=True, eos_tokens=[127],
                    model_inputs={"pixel_values": 1.0 - pix, "pixel_position_ids": pos})
    assert not np.allclose(out.logprobs[0], other.logprobs[0])


def test_sft_step_on_a_multimodal_batch():
    """The default SFT loss forwards the image arrays of a batch to a multimodal model; gradients reach the vision
    encoder and the step changes its weights."""
    from tunix_b200 import optim
    from tunix_b200.common.configs import TrainingConfig
    from tunix_b200.models.gemma4 import Gemma4Config
    from tunix_b200.models.gemma4_vision import Gemma4Multimodal, Gemma4VisionConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.sft.peft_trainer import PeftTrainer
    IMG = 120
    lm = create_model(Gemma4Config._base(vocab_size=128, embed_dim=64, hidden_dim=96, num_layers=2, num_heads=2, num_kv_heads=1,
                                         head_dim=16, global_head_dim=32, sliding_window=8, max_position=64,
                                         layer_pattern=("local", "global"), dtype=torch.float32), seed=0)
    mm = Gemma4Multimodal(lm, Gemma4VisionConfig(hidden_size=32, intermediate_size=48, num_layers=1, num_heads=2, num_kv_heads=2,
                                                 head_dim=16, patch_size=4, position_embedding_size=64, pooling_kernel_size=2,
                                                 image_token_id=IMG, dtype=torch.float32)).init_encoder_weights(seed=2, std=0.1)
    tr = PeftTrainer(mm, optim.AdamW(1e-2), TrainingConfig(eval_every_n_steps=10 ** 9, pbar_description=None,
                                                           resume_from_checkpoint_on_init=False))
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(1, 100, (2, 16), generator=g)
    toks[:, 2:6] = IMG
    batch = {"input_tokens": toks, "input_mask": (toks != IMG).float(),
             "pixel_values": torch.rand(2, 16, 48, generator=g),
             "pixel_position_ids": torch.tensor([[x, y] for y in range(4) for x in range(4)])[None].expand(2, 16, 2)}
    before = mm.vision_tower.patch_embedder.input_proj.weight.detach().clone()
    metric, _, gnorm = tr._train_step(batch, True)
    assert torch.isfinite(metric.value()) and float(gnorm) > 0
    assert not torch.equal(before, mm.vision_tower.patch_embedder.input_proj.weight.detach())
