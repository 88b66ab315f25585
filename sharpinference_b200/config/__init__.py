"""Typed configurations read from a model folder's config.json."""
from .base import ConfigError, ConfigReader, architecture_name, read_config_json
from .llama4 import Llama4TextConfig, RopeScaling

__all__ = ["ConfigError", "ConfigReader", "architecture_name", "read_config_json",
           "Llama4TextConfig", "RopeScaling"]
