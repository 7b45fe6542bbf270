from .engine_options import EngineOptions
from .model_config import (Architecture, ConfigError, LlamaConfig, get_architecture, load_config,
                           parse_config, register_architecture, registered_architectures)

__all__ = ["Architecture", "ConfigError", "EngineOptions", "LlamaConfig", "get_architecture",
           "load_config", "parse_config", "register_architecture", "registered_architectures"]
