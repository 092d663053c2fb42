"""What every part has in common, and what a mixer may ask of the cache.

A part is built from its :class:`~inferflux_b200.config.spec.PartSpec`
parameters alone: it never sees the architecture's name or configuration.  It
declares the tensors it wants (:meth:`Part.weight_specs`), receives them once
(:meth:`Part.load`, where it may fuse or re-lay them), and is then called by
the step function.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..weights.loader import WeightSpec


@dataclass(frozen=True)
class KVNeed:
    """Keys and values in pages: per token ``n_kv_heads * head_dim`` keys and as
    many values; ``window`` None = every key is kept, w = only the last w."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size, kept in the request's state slot."""

    name: str
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class PartialSums:
    """A value given as float32 slices ``[S, N, H]`` whose sum it is.  A mixer
    or feed-forward may return one instead of a tensor; the norm that follows
    adds the slices (in index order) while it adds the residual."""

    def __init__(self, tensor: torch.Tensor):
        self.tensor = tensor
        self.count = tensor.shape[0]


class Part:
    """Base of all parts.  ``params`` are the PartSpec's parameters, ``prefix``
    the weight-name prefix of the enclosing layer ("" at model level)."""

    family = ""

    def __init__(self, params: Dict[str, Any], prefix: str, dtype: torch.dtype, device: str):
        self.params = dict(params)
        self.prefix = prefix
        self.dtype = dtype
        self.device = device

    # -- naming ---------------------------------------------------------
    @staticmethod
    def full_name(prefix: str, params: Dict[str, Any], leaf: str = "") -> str:
        parts = [p for p in (prefix, params.get("name", ""), leaf) if p]
        return ".".join(parts)

    # -- weights --------------------------------------------------------
    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        return []

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Take the tensors named by :meth:`weight_specs` (those that exist)."""

    # -- cache ----------------------------------------------------------
    @classmethod
    def kv_need(cls, params: Dict[str, Any]) -> Optional[KVNeed]:
        return None

    @classmethod
    def state_needs(cls, params: Dict[str, Any]) -> List[StateNeed]:
        return []


@dataclass
class RunInfo:
    """Where one run of a layer finds its cache.

    kv_group / kv_index: the cache group and the run's place in it (None for a
    mixer without paged keys and values); writes_kv False = reads another
    run's cache.  states: the run's per-request state tensors
    ``[max_seqs, *shape]`` by name."""

    run_index: int
    kv_group: Optional[int] = None
    kv_index: Optional[int] = None
    writes_kv: bool = True
    states: Optional[Dict[str, torch.Tensor]] = None
