"""Typed configurations, read from each architecture's own config.json keys."""
from .reader import ConfigError, KeyReader, read_config_json
from .llama import LlamaConfig, Llama3RopeScaling
from .presets import preset, preset_names

__all__ = ["ConfigError", "KeyReader", "read_config_json", "LlamaConfig", "Llama3RopeScaling", "preset", "preset_names"]
