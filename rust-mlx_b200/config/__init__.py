from .base import ConfigError, ModelConfig, read_config_json
from .qwen3 import Qwen3Config
from .resolorn import ResolornConfig
from .gugalorn import GugalornConfig
from .sosuvik import SosuvikConfig
from .reverax import ReveraxConfig

__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "ResolornConfig", "GugalornConfig", "SosuvikConfig", "ReveraxConfig", "read_config_json"]
