from .model_config import ConfigError, KesozenConfig, Qwen3Config, RakizenConfig, TofilornConfig, read_config_json, write_config_json
from .engine_options import EngineOptions

__all__ = ["ConfigError", "KesozenConfig", "Qwen3Config", "RakizenConfig", "TofilornConfig", "EngineOptions", "read_config_json", "write_config_json"]
