"""Typed configurations and the architecture registry."""
from .base import ConfigError, read_config_json
from .llama import LlamaConfig, RopeScaling
from .registry import Architecture, load_config, register_architecture, resolve_architecture, supported_architectures

__all__ = [
    "Architecture",
    "ConfigError",
    "LlamaConfig",
    "RopeScaling",
    "load_config",
    "read_config_json",
    "register_architecture",
    "resolve_architecture",
    "supported_architectures",
]
