from .base import ConfigError, ModelConfig, load_config_dict
from .engine_config import EngineConfig
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "ModelConfig", "EngineConfig", "Qwen3Config", "load_config_dict"]
