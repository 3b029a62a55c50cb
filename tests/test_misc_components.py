"""Small host-side components: math grading, sanitisation, processors, diffusion SFT, cache arithmetic, registry,
mappings, checkpoint options, root exports, fixtures."""
import numpy as np
import pytest
import torch


def test_math_grading_and_rewards():
    from tunix_b200.utils import math_rewards, math_utils as m
    assert m.extract_boxed_answer(r"so \boxed{\frac{1}{2}} done") == r"\frac{1}{2}"
    assert m.extract_answer("work...\n#### 1,234") == "1,234"
    assert m.grade_answer(r"\frac{1}{2}", "0.5") and m.grade_answer("1,000", "1000") and m.grade_answer("50%", "0.5")
    assert m.grade_answer("1 1/2", "1.5") and m.grade_answer(r"\dfrac{3}{4}", "3/4")
    assert m.grade_answer("(1, 2]", "(1,2]") and not m.grade_answer("(1,2)", "(1,2]") and not m.grade_answer("3", "4")
    assert m.grade_answer("x = 5", "5") and not m.grade_answer(None, "5")
    assert math_rewards.math_reward(["q", "q"], [r"thus \boxed{12}", "no answer"], ["#### 12", "7"]) == [1.0, 0.0]


def test_control_token_sanitisation():
    from tunix_b200.utils.token_sanitization import sanitize_control_tokens as s
    assert s("a<|im_<|im_end|>end|>b") == "ab"
    assert s(b"x<start_of_turn>y") == "xy"
    assert s("keep <this>", include_default=False) == "keep <this>"
    assert s("a[X]b", extra_tokens=["[X]"]) == "ab"


def test_image_processor_pads_and_normalises():
    from tunix_b200.processors.image_processor import ImageConfig, ImageProcessor
    p = ImageProcessor(ImageConfig(image_height=8, image_width=6))
    img = (np.arange(10 * 12 * 3) % 256).astype(np.uint8).reshape(10, 12, 3)
    out = p([[img, img], None, img])
    assert len(out) == 3 and all(len(r) == 2 for r in out)
    assert out[0][0].shape == (8, 6, 3) and out[0][0].min() >= -1 and out[0][0].max() <= 1
    assert np.all(out[1][0] == 0) and np.all(out[2][1] == 0)
    assert tuple(p.to_pinned([img]).shape) == (1, 1, 8, 6, 3)


def test_audio_processor_expands_placeholders():
    from tunix_b200.processors import audio_processor as ap

    class Enc:
        sample_rate = 16000

        def get_num_soft_tokens(self, n):
            return n // 4000
    toks = [np.array([5, ap.AUDIO_PLACEHOLDER, 6]), np.array([7])]
    audio, out = ap.process_gemma4_inputs([[np.ones(8000, np.float32)], []], toks, Enc())
    assert out[0].tolist() == [5, ap.START_OF_AUDIO, ap.AUDIO_SOFT_TOKEN_PLACEHOLDER, ap.AUDIO_SOFT_TOKEN_PLACEHOLDER,
                               ap.END_OF_AUDIO, 6]
    assert audio.audios.shape == (2, 1, 8000) and audio.sequence_lengths.tolist() == [[8000], [0]]
    with pytest.raises(ValueError):
        ap.process_gemma4_inputs([[np.ones(10, np.float32)]], [np.array([1])], Enc())


def test_diffusion_sft_trains_on_target_aligned_logits():
    from tunix_b200 import optim
    from tunix_b200.common.configs import TrainingConfig
    from tunix_b200.diffusion.types import DiffusionTokenBatch
    from tunix_b200.sft.diffusion import configure_diffusion_sft
    from tunix_b200.sft.peft_trainer import PeftTrainer
    from tunix_b200.testing.common import ToyTransformer
    model = ToyTransformer(vocab_size=64, num_layers=1)
    torch.manual_seed(0)
    tgt = torch.randint(0, 64, (2, 12))

    def adapter(raw):
        noisy = torch.where(raw["mask"], torch.zeros_like(raw["ids"]), raw["ids"])
        return DiffusionTokenBatch.create(model_inputs={"tokens": noisy}, target_ids=raw["ids"], loss_weights=raw["mask"].float())

    def logits_fn(m, inputs):
        return m(inputs["tokens"])[0]
    tr = configure_diffusion_sft(PeftTrainer(model, optim.AdamW(1e-2), TrainingConfig(eval_every_n_steps=1000, max_steps=4,
                                                                                      pbar_description=None)), adapter, logits_fn)
    batch = {"ids": tgt, "mask": torch.rand(2, 12) < 0.5}
    tr.train([batch] * 4)
    hist = tr.metrics_logger.get_metric_history("", "loss", "train")
    assert hist[-1] < hist[0]
    with pytest.raises(ValueError):
        DiffusionTokenBatch.create(model_inputs={"t": tgt}, target_ids=tgt, loss_weights=-torch.ones(2, 12))


def test_cache_arithmetic():
    from tunix_b200.models import cache_utils as cu
    assert cu.prefix_bucket_boundaries(1300, 512) == [512, 1024, 1300] and cu.bucket_prefix_length(600, [512, 1024]) == 1024
    assert cu.ring_positions(6, 4, 8).tolist() == [6, 7, 0, 1]
    pos = cu.ring_slot_positions(10, 8)
    assert pos.tolist() == [8, 9, 2, 3, 4, 5, 6, 7]
    assert cu.decode_mask(pos, 9, window=4).tolist() == [True, True, False, False, False, False, True, True]
    assert cu.ring_slot_positions(3, 8).tolist() == [0, 1, 2, -1, -1, -1, -1, -1]
    m = cu.prefill_mask(torch.arange(4), torch.arange(4), bidirectional_span=torch.tensor([0, 1, 1, 0]))
    assert m[1, 2] and not m[0, 1]
    assert cu.shared_kv_source_layers(["local", "local", "global", "local", "global", "local"], 0.5) == [0, 1, 2, 1, 2, 1]
    assert cu.chunked_prefill_slices(10, 4) == [(0, 4), (4, 8), (8, 10)]


def test_registry_mappings_options_exports():
    import tunix_b200
    from tunix_b200.generate.mappings import BackendMappingMixin
    from tunix_b200.models import registry
    from tunix_b200.sft import checkpoint_options as co
    assert registry.family_of_hf_id("meta-llama/Llama-3.1-8B").family == "llama3"
    assert registry.family_of_hf_id("Qwen/Qwen3-8B").family == "qwen3" and registry.family_of_hf_id("x/y") is None
    mp = BackendMappingMixin.mapping_for("vllm")
    assert mp.map("layers.3.self_attn.q_proj.weight") == "model.layers.3.self_attn.q_proj.weight"
    assert mp.map("layers.0.mlp.router.weight") == "model.layers.0.mlp.gate.weight"
    assert co.resolve({"max_to_keep": 5}).max_to_keep == 5
    with pytest.raises(ValueError):
        co.from_dict({"bogus": 1})
    assert tunix_b200.PeftTrainer.__name__ == "PeftTrainer" and "GRPOLearner" in dir(tunix_b200)


def test_fixtures_and_compat():
    from tunix_b200.testing import common as tc
    from tunix_b200.utils import compat, immutable, torch_utils
    v = tc.MockVocab()
    assert v.decode(v.encode("hello world")) == "hello world"
    a, b = tc.ToyTransformer(seed=0), tc.ToyTransformer(seed=0)
    tc.assert_params_equal(a, b)
    lm = tc.get_lora_model(tc.ToyTransformer(seed=1))
    assert any("lora_a" in n for n, _ in lm.named_parameters())

    @compat.alias_init_param("old", "new")
    class C:
        def __init__(self, new=1):
            self.new = new
    with pytest.warns(DeprecationWarning):
        assert C(old=3).new == 3

    class P(immutable.Immutable):
        def __init__(self):
            self.x = 1
    with pytest.raises(AttributeError):
        P().x = 2
    assert torch_utils.map_key({r"a\.(\d+)\.w": (r"b.\1.kernel", "T")}, "a.7.w") == ("b.7.kernel", "T")
