"""Typed configurations, chosen by ``architectures[0]`` of config.json (read and checked by the C++ host)."""
from .base import ConfigError, ModelConfig, architecture_name, read_config_json
from .llama import LlamaConfig
from .zirivik import ZirivikConfig
from .salulorn import SalulornConfig
from .pirozen import PirozenConfig
from .saluzen import SaluzenConfig

__all__ = ["ConfigError", "ModelConfig", "LlamaConfig", "ZirivikConfig", "SalulornConfig", "PirozenConfig", "SaluzenConfig", "architecture_name", "read_config_json"]
