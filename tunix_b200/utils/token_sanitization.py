"""Scrub model control tokens out of untrusted text before it is templated into a prompt.

A user message that contains `<|im_start|>system` or `<start_of_turn>` could otherwise open a turn of its
own. Removal repeats until nothing changes, so a token hidden inside another one (`<|im_<|im_end|>end|>`)
does not survive. Behaviour of tunix/utils/token_sanitization.py:37-88.
"""
from __future__ import annotations

import re
from typing import Iterable, Optional

CONTROL_TOKENS = (
    "<|im_start|>", "<|im_end|>", "<|endoftext|>", "<|begin_of_text|>", "<|end_of_text|>", "<|start_header_id|>",
    "<|end_header_id|>", "<|eot_id|>", "<|eom_id|>", "<|python_tag|>", "<start_of_turn>", "<end_of_turn>", "<bos>", "<eos>",
    "<pad>", "<s>", "</s>", "<unk>", "<|system|>", "<|user|>", "<|assistant|>", "<|tool|>", "<tool_call>", "</tool_call>",
    "<tool_response>", "</tool_response>", "<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<start_of_image>",
    "<end_of_image>", "<|fim_prefix|>", "<|fim_middle|>", "<|fim_suffix|>", "[INST]", "[/INST]", "<<SYS>>", "<</SYS>>",
)
_DEFAULT_RE = re.compile("|".join(re.escape(t) for t in sorted(CONTROL_TOKENS, key=len, reverse=True)))


def sanitize_control_tokens(content, extra_tokens: Optional[Iterable[str]] = None, include_default: bool = True):
    if isinstance(content, memoryview):
        content = content.tobytes()
    if isinstance(content, (bytes, bytearray)):
        content = bytes(content).decode("utf-8", errors="replace")
    elif content is not None and not isinstance(content, str):
        content = str(content)
    if not content:
        return content
    extra = [t for t in (extra_tokens or ()) if t]
    if include_default and not extra:
        pattern = _DEFAULT_RE
    else:
        toks = set(extra) | (set(CONTROL_TOKENS) if include_default else set())
        if not toks:
            return content
        pattern = re.compile("|".join(re.escape(t) for t in sorted(toks, key=len, reverse=True)))
    while True:
        cleaned = pattern.sub("", content)
        if cleaned == content:
            return cleaned
        content = cleaned
