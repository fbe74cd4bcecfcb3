from .base import ConfigError, ModelConfig, read_config_json, read_generation_eos
from .qwen2 import Qwen2Config, qwen2_blueprint

__all__ = ["ConfigError", "ModelConfig", "read_config_json", "read_generation_eos", "Qwen2Config", "qwen2_blueprint"]
