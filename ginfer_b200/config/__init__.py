from .engine_config import EngineConfig
from .model_config import ConfigError, Qwen2Config, read_config_json
from .registry import (load_model_config, register_architecture, registered_architectures,
                       resolve_architecture)
