from .model_config import ConfigError, ModelConfig, read_config_json, write_config_json
from .qwen3_config import Qwen3Config
from .engine_config import EngineConfig, parse_dtype
from .presets import PRESETS, preset_config_dict, preset_init

__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "read_config_json",
           "write_config_json", "EngineConfig", "parse_dtype", "PRESETS",
           "preset_config_dict", "preset_init"]
