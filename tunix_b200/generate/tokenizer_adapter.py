"""Uniform tokenizer interface over SentencePiece, HuggingFace and duck-typed tokenizers
(tunix/generate/tokenizer_adapter.py:34-307): `encode / decode / bos_id / eos_id / pad_id /
dedup_bos_ids / apply_chat_template`."""
from __future__ import annotations

import enum
import inspect
from typing import Any, Optional, Sequence


class TokenizerType(enum.Enum):
    SP = "sp"
    HF = "hf"
    HFP = "hf_processor"
    NONE = "none"


_GEMMA_TEMPLATE_USER = "<start_of_turn>user\n{content}<end_of_turn>\n"
_GEMMA_TEMPLATE_MODEL = "<start_of_turn>model\n{content}<end_of_turn>\n"


class TokenizerAdapter:
    def __init__(self, tokenizer: Any):
        self._tokenizer = tokenizer
        mod = type(tokenizer).__module__ or ""
        if "sentencepiece" in mod:
            self._type = TokenizerType.SP
        elif "transformers" in mod or "tokenizers" in mod:
            self._type = TokenizerType.HFP if hasattr(tokenizer, "tokenizer") and not hasattr(tokenizer, "encode") \
                else TokenizerType.HF
        else:
            missing = [m for m in ("encode", "decode", "bos_id", "eos_id", "pad_id") if not hasattr(tokenizer, m)]
            if missing:
                raise AttributeError(f"Your tokenizer must implement {missing} to be used as a custom tokenizer")
            self._type = TokenizerType.NONE

    @property
    def tokenizer(self):
        return self._tokenizer

    def encode(self, text: str, **kwargs) -> list[int]:
        if self._type == TokenizerType.SP:
            return self._tokenizer.EncodeAsIds(text, **kwargs)
        if self._type == TokenizerType.HFP:
            return self._tokenizer.tokenizer.encode(text, **kwargs)
        if self._type == TokenizerType.HF:
            kwargs.setdefault("add_special_tokens", False)
            return self._tokenizer.encode(text, **kwargs)
        return self._tokenizer.encode(text, **kwargs)

    def decode(self, ids: Sequence[int], **kwargs) -> str:
        ids = [int(i) for i in ids]
        if self._type == TokenizerType.SP:
            return self._tokenizer.DecodeIds(ids, **kwargs)
        if self._type == TokenizerType.HFP:
            return self._tokenizer.tokenizer.decode(ids, **kwargs)
        return self._tokenizer.decode(ids, **kwargs)

    def _hf(self):
        return self._tokenizer.tokenizer if self._type == TokenizerType.HFP else self._tokenizer

    def bos_id(self) -> Optional[int]:
        if self._type == TokenizerType.SP:
            return self._tokenizer.bos_id()
        if self._type in (TokenizerType.HF, TokenizerType.HFP):
            return self._hf().bos_token_id
        return self._tokenizer.bos_id()

    def eos_id(self) -> Optional[int]:
        if self._type == TokenizerType.SP:
            return self._tokenizer.eos_id()
        if self._type in (TokenizerType.HF, TokenizerType.HFP):
            return self._hf().eos_token_id
        return self._tokenizer.eos_id()

    def pad_id(self) -> int:
        """Falls back to EOS (HF) or 0 when no pad token is defined."""
        if self._type == TokenizerType.SP:
            pid = self._tokenizer.pad_id()
            return pid if pid is not None and pid >= 0 else 0
        if self._type in (TokenizerType.HF, TokenizerType.HFP):
            hf = self._hf()
            if hf.pad_token_id is None:
                return hf.eos_token_id if hf.eos_token_id is not None else 0
            return hf.pad_token_id
        return self._tokenizer.pad_id()

    def dedup_bos_ids(self, ids: list[int]) -> list[int]:
        """Collapse a run of leading BOS tokens to a single one."""
        bos = self.bos_id()
        i = 0
        while i + 1 < len(ids) and ids[i] == bos and ids[i + 1] == bos:
            i += 1
        return list(ids[i:])

    def apply_chat_template(self, messages: list[dict], add_generation_prompt: bool = True, tokenize: bool = False,
                            **kwargs):
        if self._type in (TokenizerType.HF, TokenizerType.HFP) and getattr(self._hf(), "chat_template", None):
            return self._hf().apply_chat_template(messages, add_generation_prompt=add_generation_prompt,
                                                  tokenize=tokenize, **kwargs)
        if hasattr(self._tokenizer, "apply_chat_template") and self._type == TokenizerType.NONE:
            return self._tokenizer.apply_chat_template(messages, add_generation_prompt=add_generation_prompt,
                                                       tokenize=tokenize, **kwargs)
        # Gemma-style fallback template
        out = ""
        for m in messages:
            role = m.get("role", "user")
            tpl = _GEMMA_TEMPLATE_MODEL if role in ("assistant", "model") else _GEMMA_TEMPLATE_USER
            content = m.get("content", "")
            if role == "system":
                content = f"{content}\n"
            out += tpl.format(content=content)
        if add_generation_prompt:
            out += "<start_of_turn>model\n"
        return self.encode(out) if tokenize else out


class Tokenizer(TokenizerAdapter):
    """Build a tokenizer from a path: `tokenizer_type` in {"sentencepiece", "huggingface"}."""

    def __init__(self, tokenizer_type: str = "sentencepiece", tokenizer_path: str = "", add_bos: bool = True,
                 add_eos: bool = True, hf_access_token: Optional[str] = None):
        self.add_bos, self.add_eos = add_bos, add_eos
        if tokenizer_type == "huggingface":
            from transformers import AutoTokenizer
            tok = AutoTokenizer.from_pretrained(tokenizer_path, token=hf_access_token)
        elif tokenizer_type == "sentencepiece":
            import sentencepiece as spm
            tok = spm.SentencePieceProcessor()
            tok.Load(tokenizer_path)
        else:
            raise ValueError(f"Unsupported tokenizer_type: {tokenizer_type}")
        super().__init__(tok)

    def tokenize(self, example: str, prefix: str = "", suffix: str = "", add_eos: bool = True) -> list[int]:
        ids = []
        if self.add_bos and self.bos_id() is not None:
            ids.append(self.bos_id())
        ids += self.encode(prefix + example + suffix)
        if self.add_eos and add_eos and self.eos_id() is not None:
            ids.append(self.eos_id())
        return ids
