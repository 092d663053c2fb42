"""Registries: architecture name -> (typed config, spec builder), and part
kind -> part class for mixers, feed-forwards, norms, position encodings,
block arrangements, embeddings and output heads.

The reference keys its only forward class on the lower-cased ``model_type``
(runtime/backends/cuda/native/model_forward_factory.cpp:13-25,34-48), so a
config that carries only ``architectures: ["Qwen2ForCausalLM"]`` is rejected
there.  Here ``architectures[0]`` is looked up first and ``model_type`` second.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Tuple, Type

from .model_config import ConfigError, ModelConfig, read_config_dict
from .spec import ModelSpec

_ARCHITECTURES: Dict[str, Tuple[Type[ModelConfig], Callable[[Any], ModelSpec]]] = {}
_ALIASES: Dict[str, str] = {}

PART_FAMILIES = ("mixer", "feed_forward", "norm", "position", "arrangement",
                 "embedding", "lm_head")
_PARTS: Dict[str, Dict[str, type]] = {fam: {} for fam in PART_FAMILIES}


def register_architecture(name: str, config_cls: Type[ModelConfig],
                          build_spec: Callable[[Any], ModelSpec],
                          model_type: str = "") -> None:
    _ARCHITECTURES[name] = (config_cls, build_spec)
    if model_type:
        _ALIASES[model_type.lower()] = name


def resolve_architecture(config_dict: Dict[str, Any]) -> str:
    _ensure_builtin()
    archs = config_dict.get("architectures") or []
    for a in archs:
        if a in _ARCHITECTURES:
            return a
    mt = str(config_dict.get("model_type", "") or "").lower()
    if mt in _ALIASES:
        return _ALIASES[mt]
    known = ", ".join(sorted(_ARCHITECTURES)) or "(none)"
    raise ConfigError(
        f"no registered architecture for architectures={archs!r}, "
        f"model_type={config_dict.get('model_type')!r}; known: {known}")


def load_config(folder_or_dict) -> ModelConfig:
    d = folder_or_dict if isinstance(folder_or_dict, dict) else read_config_dict(folder_or_dict)
    name = resolve_architecture(d)
    config_cls, _ = _ARCHITECTURES[name]
    return config_cls.from_dict(d)


def build_spec(config: ModelConfig) -> ModelSpec:
    _ensure_builtin()
    for name, (config_cls, builder) in _ARCHITECTURES.items():
        if type(config) is config_cls:
            spec = builder(config)
            spec.validate()
            return spec
    raise ConfigError(f"no architecture registered for config type {type(config).__name__}")


def register_part(family: str, kind: str, cls: type) -> None:
    if family not in _PARTS:
        raise KeyError(f"unknown part family '{family}'; one of {PART_FAMILIES}")
    _PARTS[family][kind] = cls


def part_class(family: str, kind: str) -> type:
    _ensure_builtin()
    try:
        return _PARTS[family][kind]
    except KeyError:
        known = ", ".join(sorted(_PARTS.get(family, {}))) or "(none)"
        raise KeyError(f"no {family} part of kind '{kind}' is registered; known: {known}") from None


def registered_architectures():
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


_builtin_loaded = False


def _ensure_builtin() -> None:
    """Import the modules that register the built-in parts and architecture."""
    global _builtin_loaded
    if _builtin_loaded:
        return
    _builtin_loaded = True
    from .. import parts  # noqa: F401  (registers parts)
    from .. import models  # noqa: F401  (registers architectures)
