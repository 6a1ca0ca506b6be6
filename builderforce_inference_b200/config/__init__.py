from .base import ConfigError, ConfigReader, read_json, stop_ids_of_folder
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "ConfigReader", "Qwen3Config", "read_json", "stop_ids_of_folder"]
