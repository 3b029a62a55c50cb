"""Qwen 2.5 (and the DeepSeek-R1 distillations on it): family entry points over the shared decoder."""
from . import model, params  # noqa: F401
