from .engine_config import EngineConfig, add_engine_args, engine_config_from_args
from .kutirax_config import KutiraxConfig
from .model_config import ConfigError, Qwen2Config, architecture_name, read_config_json

__all__ = ["EngineConfig", "add_engine_args", "engine_config_from_args", "ConfigError", "Qwen2Config",
           "KutiraxConfig", "architecture_name", "read_config_json"]
