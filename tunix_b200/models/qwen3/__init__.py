"""Qwen 3 (dense and mixture-of-experts): family entry points over the shared decoder."""
from . import model, params  # noqa: F401
