from .base import ConfigError, read_config_json
from .qwen2 import Qwen2Config

__all__ = ["ConfigError", "Qwen2Config", "read_config_json"]
