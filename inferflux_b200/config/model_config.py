"""Typed model configuration read from an architecture's own ``config.json`` keys.

The reference parses the same keys into ``SafetensorsLoader::ModelConfig``
(runtime/backends/cuda/inferflux_cuda_executor.h:62-85, parse at
runtime/backends/cuda/inferflux_cuda_executor.cpp:524-604): ``hidden_size``,
``num_hidden_layers``, ``num_attention_heads``, ``num_key_value_heads``,
``head_dim`` (default ``hidden_size / num_attention_heads``),
``intermediate_size``, ``vocab_size``, ``max_position_embeddings``,
``rope_theta`` (default 10000), ``rms_norm_eps`` (default 1e-6),
``model_type`` / ``architectures``, ``hidden_act``, ``torch_dtype``.
It silently keeps defaults when the file cannot be parsed
(inferflux_cuda_executor.cpp:348-351); here every fault is an error.

Keys the reference never reads but the architecture defines
(``tie_word_embeddings``, ``use_sliding_window``, ``sliding_window``,
``max_window_layers``, ``bos_token_id``, ``eos_token_id``) are typed here too.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that cannot describe a runnable model."""


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's typed configuration."""

    architectures: List[str] = field(default_factory=list)
    model_type: str = ""

    @property
    def architecture(self) -> str:
        if self.architectures:
            return self.architectures[0]
        return self.model_type

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    def save(self, folder: str) -> str:
        os.makedirs(folder, exist_ok=True)
        path = os.path.join(folder, "config.json")
        with open(path, "w") as f:
            json.dump(self.to_dict(), f, indent=2, sort_keys=True)
        return path


def _require_int(d: Dict[str, Any], key: str, minimum: int = 1) -> int:
    if key not in d:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: '{key}' must be >= {minimum}, got {v}")
    return v


def _opt_number(d: Dict[str, Any], key: str, default: float) -> float:
    v = d.get(key, default)
    if v is None:
        return float(default)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    """``Qwen2ForCausalLM``: pre-norm RMSNorm decoder, grouped-query attention
    with q/k/v bias, rotate-half rotary positions, SwiGLU feed-forward."""

    hidden_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    vocab_size: int = 0
    max_position_embeddings: int = 0
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None

    ARCHITECTURE = "Qwen2ForCausalLM"
    MODEL_TYPE = "qwen2"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen2Config":
        archs = d.get("architectures") or []
        if not isinstance(archs, list):
            raise ConfigError("config.json: 'architectures' must be a list")
        model_type = d.get("model_type", "") or ""
        hidden = _require_int(d, "hidden_size")
        heads = _require_int(d, "num_attention_heads")
        # The reference leaves num_key_value_heads at 0 when absent
        # (inferflux_cuda_executor.cpp:537-539); multi-head attention is the
        # meaning of an absent key, so that is the default here.
        kv_heads = _require_int(d, "num_key_value_heads") if "num_key_value_heads" in d else heads
        if "head_dim" in d and d["head_dim"] is not None:
            head_dim = _require_int(d, "head_dim")
        else:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not divisible by "
                    f"num_attention_heads {heads} and 'head_dim' is not given")
            head_dim = hidden // heads
        rope_scaling = d.get("rope_scaling")
        if rope_scaling not in (None, {}):
            raise ConfigError(
                f"config.json: rope_scaling={rope_scaling!r} is not supported "
                "(only unscaled rotary positions)")
        act = d.get("hidden_act", "silu")
        use_sw = bool(d.get("use_sliding_window", False))
        sw = d.get("sliding_window")
        if sw is not None and (isinstance(sw, bool) or not isinstance(sw, int) or sw < 1):
            raise ConfigError(f"config.json: 'sliding_window' must be a positive integer, got {sw!r}")
        layers = _require_int(d, "num_hidden_layers")
        mwl = d.get("max_window_layers", layers)
        if mwl is None:
            mwl = layers
        eos = d.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        cfg = cls(
            architectures=list(archs),
            model_type=model_type,
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=_require_int(d, "intermediate_size"),
            vocab_size=_require_int(d, "vocab_size"),
            max_position_embeddings=_require_int(d, "max_position_embeddings"),
            rope_theta=_opt_number(d, "rope_theta", 10000.0),
            rms_norm_eps=_opt_number(d, "rms_norm_eps", 1e-6),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            use_sliding_window=use_sw,
            sliding_window=sw,
            max_window_layers=int(mwl),
            hidden_act=str(act),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16")) or "bfloat16"),
            bos_token_id=d.get("bos_token_id"),
            eos_token_id=eos,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary positions")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act '{self.hidden_act}' is not supported (silu only)")
        if self.rope_theta <= 0:
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        if self.rms_norm_eps <= 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if self.use_sliding_window and not self.sliding_window:
            raise ConfigError("use_sliding_window is true but 'sliding_window' is not given")
        if not 0 <= self.max_window_layers:
            raise ConfigError("max_window_layers must be >= 0")

    def window_of_layer(self, layer: int) -> Optional[int]:
        """The attention window of a layer, or None for all keys.

        Layers from ``max_window_layers`` upwards look at the last
        ``sliding_window`` keys (the query's own included) when
        ``use_sliding_window`` is set; the layers below see every key.
        """
        if self.use_sliding_window and self.sliding_window and layer >= self.max_window_layers:
            return int(self.sliding_window)
        return None


def read_config_dict(folder_or_file: str) -> Dict[str, Any]:
    path = folder_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json at {path}")
    try:
        with open(path) as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d
