"""Typed configurations, read from each architecture's own config.json keys."""
from .llama import ConfigError, LlamaConfig, RopeScaling  # noqa: F401
