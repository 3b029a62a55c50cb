"""Parameter-name mappings towards external serving engines (tunix/generate/mappings.py:1-174).

The in-framework engine reads the trainer's parameters directly, so no mapping is needed for rollout. The table
here serves export: it maps this framework's names to the Hugging Face names a vLLM / SGLang server loads, and
is what `safetensors_saver` and a custom `rl.reshard.WeightReshard(key_map=...)` consult.
"""
from __future__ import annotations

import dataclasses
import re
from typing import Optional


@dataclasses.dataclass(frozen=True)
class MappingConfig:
    to_hf: dict                      # regex over our names -> HF template
    lora_to_hf: Optional[dict] = None
    tied_head: bool = False

    def map(self, name: str) -> str:
        for pat, tmpl in self.to_hf.items():
            m = re.fullmatch(pat, name)
            if m:
                return m.expand(tmpl)
        raise KeyError(f"no mapping for parameter {name!r}")


_DECODER = {
    r"embed_tokens": "model.embed_tokens.weight",
    r"lm_head": "lm_head.weight",
    r"norm\.weight": "model.norm.weight",
    r"layers\.(\d+)\.(input_layernorm|post_attention_layernorm|post_attn_norm|post_ffw_norm)\.weight": r"model.layers.\1.\2.weight",
    r"layers\.(\d+)\.self_attn\.(q|k|v|o)_proj\.(weight|bias)": r"model.layers.\1.self_attn.\2_proj.\3",
    r"layers\.(\d+)\.self_attn\.(q|k)_norm\.weight": r"model.layers.\1.self_attn.\2_norm.weight",
    r"layers\.(\d+)\.mlp\.(gate|up|down)_proj\.weight": r"model.layers.\1.mlp.\2_proj.weight",
    r"layers\.(\d+)\.mlp\.router\.weight": r"model.layers.\1.mlp.gate.weight",
}


class BackendMappingMixin:
    """Models expose `mapping_for(backend)`; every backend that loads Hugging Face checkpoints shares one table."""

    BACKENDS = ("hf", "vllm", "sglang")

    @classmethod
    def mapping_for(cls, backend: str = "hf") -> MappingConfig:
        if backend not in cls.BACKENDS:
            raise ValueError(f"unknown backend {backend!r}; known: {cls.BACKENDS}")
        return MappingConfig(dict(_DECODER))
