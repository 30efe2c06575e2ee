from .errors import ConfigError, UnsupportedConfig
from .spec import PartSpec, LayerSpec, RunEntry, ModelSpec
from .qwen3 import Qwen3Config
from .registry import Architecture, ArchitectureRegistry, default_registry, read_model_config

__all__ = [
    "ConfigError", "UnsupportedConfig", "PartSpec", "LayerSpec", "RunEntry", "ModelSpec",
    "Qwen3Config", "Architecture", "ArchitectureRegistry", "default_registry",
    "read_model_config",
]
