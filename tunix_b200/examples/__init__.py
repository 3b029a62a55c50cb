"""Data pipelines used by the example recipes."""
