"""Model / tokenizer construction for the CLI (tunix/cli/utils/model.py:31-229)."""
from __future__ import annotations

import torch

from ...lora import LoraProvider, apply_lora_to_model
from ...models.automodel import AutoModel, ModelSource
from ...generate.tokenizer_adapter import Tokenizer, TokenizerAdapter

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


class CharTokenizer:
    """Byte-level fallback tokenizer for smoke runs without tokenizer files."""

    def __init__(self, vocab_size: int = 259):
        self.vocab_size = vocab_size

    def encode(self, s, **kw):
        return [3 + b for b in s.encode("utf-8")]

    def decode(self, ids, **kw):
        return bytes([max(0, min(255, int(i) - 3)) for i in ids if int(i) >= 3]).decode("utf-8", errors="replace")

    def bos_id(self):
        return 1

    def eos_id(self):
        return 2

    def pad_id(self):
        return 0


def create_model(model_cfg: dict, device=None):
    src = ModelSource(model_cfg.get("model_source") or "random")
    dtype = _DTYPES[model_cfg.get("dtype", "bfloat16")] if (device is not None and torch.device(device).type == "cuda") \
        else torch.float32
    model, path = AutoModel.from_pretrained(
        model_cfg["model_id"], model_source=src, model_path=model_cfg.get("model_path") or None,
        model_download_path=model_cfg.get("model_download_path"), device=device, dtype=dtype,
        remat_config=model_cfg.get("remat_config"), seed=model_cfg.get("rng_seed", 0),
        **(model_cfg.get("config_overrides") or {}))
    lc = model_cfg.get("lora_config") or {}
    if lc:
        apply_lora_to_model(model, LoraProvider(module_path=lc.get("module_path", LoraProvider.module_path),
                                                rank=lc.get("rank", 8), alpha=lc.get("alpha", 16.0),
                                                weight_qtype=lc.get("weight_qtype"), tile_size=lc.get("tile_size", 64)))
    if model_cfg.get("model_display"):
        print(model)
    return model


def create_tokenizer(tok_cfg: dict):
    t = tok_cfg.get("tokenizer_type", "huggingface")
    if t == "char" or not tok_cfg.get("tokenizer_path"):
        return TokenizerAdapter(CharTokenizer())
    return Tokenizer(t, tok_cfg["tokenizer_path"], tok_cfg.get("add_bos", True), tok_cfg.get("add_eos", True))
