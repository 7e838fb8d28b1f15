from .base import ConfigError, ConfigReader, read_json
from .generation import GenerationDefaults, read_generation_defaults
from .qwen2 import Qwen2Config

__all__ = ["ConfigError", "ConfigReader", "read_json", "GenerationDefaults", "read_generation_defaults", "Qwen2Config"]
