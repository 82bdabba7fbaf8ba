from .base import ConfigError, read_config_json
from .engine import EngineConfig, KernelSwitches
from .registry import Architecture, known_architectures, load_config, register_architecture, resolve_architecture

__all__ = ["ConfigError", "EngineConfig", "KernelSwitches", "read_config_json", "Architecture", "known_architectures", "load_config",
           "register_architecture", "resolve_architecture"]
