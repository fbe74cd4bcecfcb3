from .base import ConfigError, ModelConfig, read_config_json
from .qwen2 import Qwen2Config, qwen2_blueprint

__all__ = ["ConfigError", "ModelConfig", "read_config_json", "Qwen2Config", "qwen2_blueprint"]
