"""Typed configurations and the part specs they translate into."""
from .llama import ConfigError, LlamaConfig
from . import specs

__all__ = ["ConfigError", "LlamaConfig", "specs"]
