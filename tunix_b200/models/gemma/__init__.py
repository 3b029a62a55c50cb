"""Gemma 1 and 2: family entry points over the shared decoder."""
from . import model, params  # noqa: F401
