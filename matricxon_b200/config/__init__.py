from matricxon_b200.config.base import ConfigError
from matricxon_b200.config.registry import (
    ArchitectureEntry,
    UnsupportedArchitectureError,
    config_from_dict,
    entry_for_config,
    load_config,
    register_architecture,
    resolve_architecture,
    supported_names,
)
from matricxon_b200.config.starcoder2 import Starcoder2Config

__all__ = [
    "ArchitectureEntry", "ConfigError", "Starcoder2Config", "UnsupportedArchitectureError",
    "config_from_dict", "entry_for_config", "load_config", "register_architecture",
    "resolve_architecture", "supported_names",
]
