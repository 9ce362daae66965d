from .engine_config import EngineConfig, canonical_dtype
from .model_config import ConfigError, LlamaConfig, RopeScaling, read_config_json

__all__ = ["EngineConfig", "canonical_dtype", "ConfigError", "LlamaConfig", "RopeScaling",
           "read_config_json"]
