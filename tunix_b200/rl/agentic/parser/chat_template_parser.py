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


class Gemma4ChatTemplateParser(ChatTemplateParser):
    """Gemma 4 turns (`<|turn>role\\n ... <turn|>\\n`), with the thinking switch of the family: thinking on puts
    `<|think|>` into the system turn (one is made up when the conversation has none); thinking off opens the model
    turn with an empty thought channel (tunix/rl/agentic/parser/chat_template_parser/parser.py:436-540)."""
    assistant_end = "<turn|>"

    def __init__(self, tokenizer=None, enable_thinking: bool = True):
        super().__init__(tokenizer)
        self.enable_thinking = enable_thinking
        self.generation_prompt = "<|turn>model\n" + ("" if enable_thinking else "<|channel>thought\n<channel|>")

    def parse(self, messages, add_generation_prompt: bool = False, is_first_msg: bool = True) -> str:
        out = ""
        if is_first_msg:
            out = "<bos>"
            if messages and messages[0]["role"] not in ("system", "developer") and self.enable_thinking:
                out += "<|turn>system\n<|think|><turn|>\n"
        for m in messages:
            out += self.render_message(m)
        if add_generation_prompt:
            out += self.generation_prompt
        return out

    def render_message(self, m):
        role, content = m["role"], str(m["content"]).replace("<turn|>\n", "").strip()
        if role in ("system", "developer"):
            return "<|turn>system\n" + ("<|think|>" if self.enable_thinking else "") + content + "<turn|>\n"
        if role == "tool":
            return "<|tool_response>" + str(m["content"]) + "<tool_response|>"
        if role == "assistant":
            body = str(m["content"]).strip()
            prefix = "<|turn>model\n" if self.enable_thinking else self.generation_prompt
            return prefix + body + ("\n" if body.endswith("<turn|>") else "<turn|>\n")
        return "<|turn>user\n" + content.replace("<turn|>", "") + "<turn|>\n"

    def update_assistant_end_tokens(self, tokens):
        """An assistant turn is rendered with a newline after its end token, so the sampled tokens get the same
        suffix (otherwise rollout and trainer log-probs disagree). Returns (tokens, number appended)."""
        import numpy as np
        try:
            nl = self.tokenizer.encode("\n", add_special_tokens=False)
        except TypeError:
            nl = self.tokenizer.encode("\n")
        special = set()
        for name in ("bos_id", "eos_id"):
            v = getattr(self.tokenizer, name, None)
            special.add(v() if callable(v) else v)
        nl = [t for t in nl if t not in special]
        return np.concatenate([np.asarray(tokens), np.asarray(nl, dtype=np.int32)]), len(nl)


class RawTextParser(ChatTemplateParser):
    def render_message(self, m):
        return str(m["content"])


_PARSERS = {"default": DefaultChatTemplateParser, "qwen": QwenChatTemplateParser, "llama": LlamaChatTemplateParser,
            "gemma": GemmaChatTemplateParser, "gemma4": Gemma4ChatTemplateParser, "raw": RawTextParser}


def get_parser(kind: str = "default", tokenizer=None) -> ChatTemplateParser:
    if kind not in _PARSERS:
        raise ValueError(f"unknown chat parser {kind!r}; known: {sorted(_PARSERS)}")
    return _PARSERS[kind](tokenizer)
