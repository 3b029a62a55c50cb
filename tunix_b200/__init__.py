"""tunix_b200: a Blackwell (sm_100a) native LLM post-training framework."""
__version__ = "0.1.0"
