from .model_config import ConfigError, Qwen3Config, read_config_json
from .registry import Architecture, known, lookup, read_model_config, register, unregister
