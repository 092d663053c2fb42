from .model_config import ConfigError, ModelConfig, Qwen2Config, read_config_dict
from .engine_config import EngineConfig
from .spec import PartSpec, LayerSpec, Run, ModelSpec
from .registry import (register_architecture, register_part, part_class, load_config,
                       build_spec, resolve_architecture, registered_architectures)

__all__ = [
    "ConfigError", "ModelConfig", "Qwen2Config", "read_config_dict", "EngineConfig",
    "PartSpec", "LayerSpec", "Run", "ModelSpec", "register_architecture", "register_part",
    "part_class", "load_config", "build_spec", "resolve_architecture",
    "registered_architectures",
]
