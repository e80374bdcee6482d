from .engine_config import EngineConfig
from .model_config import ConfigError, ModelConfig, Qwen3Config, read_config_json
from .registry import (Architecture, load_config, register_architecture, registered_architectures,
                       resolve_architecture, unregister_architecture)

__all__ = [
    "EngineConfig", "ConfigError", "ModelConfig", "Qwen3Config", "read_config_json", "Architecture",
    "load_config", "register_architecture", "registered_architectures", "resolve_architecture",
    "unregister_architecture",
]
