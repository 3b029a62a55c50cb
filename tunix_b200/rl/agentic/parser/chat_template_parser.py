"""Incremental chat templating (tunix/rl/agentic/parser/chat_template_parser/parser.py): render a list of
messages, optionally only the new ones (`is_first_msg=False`), with the generation prompt of the family and
the assistant end-of-turn token."""
from __future__ import annotations

from typing import Optional


class ChatTemplateParser:
    generation_prompt = ""
    assistant_end = ""

    def __init__(self, tokenizer=None):
        self.tokenizer = tokenizer

    def render_message(self, m: dict) -> str:
        raise NotImplementedError

    def parse(self, messages: list, add_generation_prompt: bool = False, is_first_msg: bool = True) -> str:
        out = self.bos() if is_first_msg else ""
        for m in messages:
            out += self.render_message(m)
        if add_generation_prompt:
            out += self.generation_prompt
        return out

    def bos(self) -> str:
        return ""


class DefaultChatTemplateParser(ChatTemplateParser):
    """Uses the tokenizer's own chat template when it has one."""

    def parse(self, messages, add_generation_prompt: bool = False, is_first_msg: bool = True) -> str:
        if self.tokenizer is not None and hasattr(self.tokenizer, "apply_chat_template"):
            return self.tokenizer.apply_chat_template(messages, add_generation_prompt=add_generation_prompt, tokenize=False)
        return super().parse(messages, add_generation_prompt, is_first_msg)

    def render_message(self, m):
        return f"{m['role']}: {m['content']}\n"

    generation_prompt = "assistant: "


class QwenChatTemplateParser(ChatTemplateParser):
    generation_prompt = "<|im_start|>assistant\n"
    assistant_end = "<|im_end|>"

    def render_message(self, m):
        role = "user" if m["role"] == "tool" else m["role"]
        content = f"<tool_response>\n{m['content']}\n</tool_response>" if m["role"] == "tool" else m["content"]
        return f"<|im_start|>{role}\n{content}<|im_end|>\n"


class LlamaChatTemplateParser(ChatTemplateParser):
    generation_prompt = "<|start_header_id|>assistant<|end_header_id|>\n\n"
    assistant_end = "<|eot_id|>"

    def bos(self):
        return "<|begin_of_text|>"

    def render_message(self, m):
        role = "ipython" if m["role"] == "tool" else m["role"]
        return f"<|start_header_id|>{role}<|end_header_id|>\n\n{m['content']}<|eot_id|>"


class GemmaChatTemplateParser(ChatTemplateParser):
    generation_prompt = "<start_of_turn>model\n"
    assistant_end = "<end_of_turn>"

    def bos(self):
        return "<bos>"

    def render_message(self, m):
        role = "model" if m["role"] == "assistant" else "user"
        return f"<start_of_turn>{role}\n{m['content']}<end_of_turn>\n"


class RawTextParser(ChatTemplateParser):
    def render_message(self, m):
        return str(m["content"])


_PARSERS = {"default": DefaultChatTemplateParser, "qwen": QwenChatTemplateParser, "llama": LlamaChatTemplateParser,
            "gemma": GemmaChatTemplateParser, "raw": RawTextParser}


def get_parser(kind: str = "default", tokenizer=None) -> ChatTemplateParser:
    if kind not in _PARSERS:
        raise ValueError(f"unknown chat parser {kind!r}; known: {sorted(_PARSERS)}")
    return _PARSERS[kind](tokenizer)
