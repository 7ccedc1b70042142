from .model_config import ConfigError, DepolixConfig, KesozenConfig, Qwen3Config, RakizenConfig, TofilornConfig, read_config_json, write_config_json
from .engine_options import EngineOptions

__all__ = ["ConfigError", "DepolixConfig", "KesozenConfig", "Qwen3Config", "RakizenConfig", "TofilornConfig", "EngineOptions", "read_config_json", "write_config_json"]
