"""Gemma 3 text: family entry points over the shared decoder."""
from . import model, params  # noqa: F401
