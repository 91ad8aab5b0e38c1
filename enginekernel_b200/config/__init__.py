"""Typed configurations, one class per architecture."""
from .base import ConfigError, ModelConfig, key, read_config_json
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "key", "read_config_json"]
