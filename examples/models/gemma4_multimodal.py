"""Gemma 4 with image and audio inputs, random weights, CPU or GPU.

    python examples/models/gemma4_multimodal.py

Builds a small Gemma-4-style decoder (per-layer inputs, KV sharing, alternating local / global layers), the vision and
audio encoders in front of it, and runs one forward pass over a prompt with image and audio placeholders. A real
checkpoint loads with `models.safetensors_loader.load_safetensors_into(language_model, path)` and
`vision_tower.load_state_dict(...)` (the module names follow the Hugging Face checkpoint)."""
import torch

from tunix_b200.models.gemma4 import Gemma4Config
from tunix_b200.models.gemma4_audio import Gemma4AudioConfig
from tunix_b200.models.gemma4_vision import Gemma4Multimodal, Gemma4VisionConfig
from tunix_b200.models.transformer import create_model


def main():
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    IMG, AUD = 250, 251
    lm = create_model(Gemma4Config._base(vocab_size=256, embed_dim=128, hidden_dim=256, num_layers=6, num_heads=2, num_kv_heads=1,
                                         head_dim=64, global_head_dim=128, sliding_window=32, max_position=256,
                                         per_layer_input_dim=16, num_kv_shared_layers=2, layer_pattern=("local", "global"),
                                         dtype=dt), device=dev, seed=0)
    vis = Gemma4VisionConfig(hidden_size=64, intermediate_size=128, num_layers=2, num_heads=1, num_kv_heads=1, head_dim=64,
                             patch_size=4, position_embedding_size=64, pooling_kernel_size=2, image_token_id=IMG, dtype=dt)
    aud = Gemma4AudioConfig(hidden_size=64, num_layers=2, num_heads=4, subsampling_conv_channels=(16, 8), output_proj_dims=48,
                            audio_token_id=AUD, dtype=dt)
    model = Gemma4Multimodal(lm, vis, audio_config=aud, device=dev).to(dev).init_encoder_weights(seed=0, std=0.05)
    # one 8 x 8-patch image -> 16 soft tokens; 64 mel frames -> 16 audio frames
    pos = torch.tensor([[x, y] for y in range(8) for x in range(8)], device=dev)[None]
    pixels = torch.rand(1, 64, 3 * 4 * 4, device=dev)
    mel = torch.randn(1, 64, 16, device=dev)
    tokens = torch.tensor([[2, 17, 18] + [IMG] * 16 + [40, 41] + [AUD] * 16 + [55, 56]], device=dev)
    with torch.no_grad():
        logits, _ = model(tokens, pixel_values=pixels, pixel_position_ids=pos, input_features=mel,
                          input_features_mask=torch.ones(1, 64, dtype=torch.bool, device=dev))
    print("logits", tuple(logits.shape), "next token", int(logits[0, -1].argmax()))


if __name__ == "__main__":
    main()
