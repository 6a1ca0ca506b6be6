from .base import ConfigError, ConfigReader, read_json
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "ConfigReader", "Qwen3Config", "read_json"]
