from .model_config import ConfigError, Qwen2Config, architecture_name, read_config_json
from .registry import (Architecture, register_architecture, unregister_architecture,
                       registered_architectures, resolve_architecture, load_config)
from .options import EngineOptions
from .fezopel_config import FezopelConfig
from .kavotar_config import KavotarConfig
from .miforax_config import MiforaxConfig
from .dapuzen_config import DapuzenConfig

__all__ = [
    "ConfigError", "Qwen2Config", "FezopelConfig", "KavotarConfig", "MiforaxConfig", "DapuzenConfig", "architecture_name", "read_config_json", "Architecture",
    "register_architecture", "unregister_architecture", "registered_architectures",
    "resolve_architecture", "load_config", "EngineOptions",
]
