"""Typed configurations: the architecture's config.json (`Qwen2Config`) and the engine's options."""
from .base import ConfigError, ConfigReader, read_config_json, architecture_name
from .qwen2 import Qwen2Config
from .engine import EngineConfig

__all__ = ["ConfigError", "ConfigReader", "read_config_json", "architecture_name", "Qwen2Config", "EngineConfig"]
