from .base import ConfigError, read_config_json
from .registry import Architecture, known_architectures, load_config, register_architecture, resolve_architecture

__all__ = ["ConfigError", "read_config_json", "Architecture", "known_architectures", "load_config",
           "register_architecture", "resolve_architecture"]
