from .base import ConfigError, read_config_json
from .engine import EngineConfig, parse_dtype
from .gemma import GemmaConfig
from .registry import ARCHITECTURES, Architecture, config_from_folder, register_architecture, resolve_architecture

__all__ = ["ConfigError", "read_config_json", "EngineConfig", "parse_dtype", "GemmaConfig", "ARCHITECTURES",
           "Architecture", "config_from_folder", "register_architecture", "resolve_architecture"]
