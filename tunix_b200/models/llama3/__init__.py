"""Llama 3.x: family entry points over the shared decoder."""
from . import model, params  # noqa: F401
