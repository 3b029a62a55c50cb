"""Small fixtures shared by tests and examples (role of tunix/tests/test_common.py): a toy vocabulary / tokenizer,
a toy decoder built from the real model code, and helpers to attach LoRA and compare parameter sets."""
from __future__ import annotations

import torch

from ..models.config import ModelConfig
from ..models.transformer import create_model


class MockVocab:
    """Word-level vocabulary with the tokenizer-adapter surface (`encode`, `decode`, ids of special tokens)."""

    def __init__(self, words=None):
        words = words or ("<pad> <s> </s> input string hello world Hello there ! My name is Morgane Tunix James Peter "
                          "quick brown fox jumps over the lazy dog one two three four five six seven eight nine ten").split()
        self._id = {w: i for i, w in enumerate(words)}
        self._word = dict(enumerate(words))

    def GetPieceSize(self) -> int:
        return len(self._id)

    vocab_size = property(lambda self: len(self._id))

    def pad_id(self) -> int:
        return 0

    def bos_id(self) -> int:
        return 1

    def eos_id(self) -> int:
        return 2

    def encode(self, text: str, **_):
        return [self._id.get(w, self._id["<pad>"]) for w in text.split()]

    EncodeAsIds = encode

    def decode(self, ids, **_):
        return " ".join(self._word.get(int(i), "<unk>") for i in ids)

    DecodeIds = decode


def toy_config(vocab_size: int = 256, num_layers: int = 2, **kw) -> ModelConfig:
    base = dict(num_layers=num_layers, vocab_size=vocab_size, embed_dim=64, hidden_dim=128, num_heads=4, head_dim=16, num_kv_heads=2)
    base.update(kw)
    return ModelConfig.tiny_llama().replace(**base)


def ToyTransformer(vocab_size: int = 256, num_layers: int = 2, seed: int = 0, device=None, **kw):
    return create_model(toy_config(vocab_size, num_layers, **kw), device=device, seed=seed)


def get_lora_model(model, rank: int = 4, alpha: float = 8.0, module_path: str = r".*(q_proj|v_proj|gate_proj|up_proj)"):
    from .. import lora
    return lora.apply_lora_to_model(model, lora.LoraProvider(module_path=module_path, rank=rank, alpha=alpha))


def assert_params_equal(a, b, atol: float = 0.0) -> None:
    pa, pb = dict(a.named_parameters()), dict(b.named_parameters())
    assert pa.keys() == pb.keys(), sorted(set(pa) ^ set(pb))
    for n in pa:
        assert torch.allclose(pa[n].float(), pb[n].float(), atol=atol), n


def assert_params_differ(a, b, names=None) -> None:
    pa, pb = dict(a.named_parameters()), dict(b.named_parameters())
    for n in (names or pa):
        assert not torch.equal(pa[n], pb[n]), f"{n} did not change"
