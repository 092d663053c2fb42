"""The description of a model as data: which parts each layer is made of and
in which order layers run.

An architecture is a function from its typed configuration to a
:class:`ModelSpec`.  Nothing below the spec knows the architecture's name: a
part gets its sizes and constants from its :class:`PartSpec` parameters.

The reference hard-wires one block shape for every model family
(runtime/backends/cuda/native/llama_forward.h:84-89) and selects it by a
``model_type`` string (runtime/backends/cuda/native/model_forward_factory.cpp:34-48);
the per-layer list here replaces that.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part: the registered ``kind`` and the parameters it is built with."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its weight-name prefix, how its parts are arranged, and the
    parts themselves by the role each plays in that arrangement.

    Which roles there are is the arrangement's business: it declares them with
    the family of part that fills each (``prenorm``: ``mixer``, ``mixer_norm``,
    ``feed_forward``, ``feed_forward_norm``); the model builds whatever the
    layer lists and hands the lot to the arrangement.  A block with more norms,
    with one norm for two parallel branches or without a feed-forward is
    another arrangement with other roles, not a change to this class.

    ``position`` names an entry of :attr:`ModelSpec.positions` (or None for a
    layer whose mixer needs no position encoding).
    """

    prefix: str
    arrangement: str
    parts: Dict[str, PartSpec]
    position: Optional[str] = None

    def part(self, role: str) -> PartSpec:
        try:
            return self.parts[role]
        except KeyError:
            raise KeyError(f"layer '{self.prefix}' has no part in the role '{role}'; "
                           f"it has {sorted(self.parts)}") from None


@dataclass(frozen=True)
class Run:
    """One entry of the execution order.

    ``layer`` indexes :attr:`ModelSpec.layers`; a layer may appear in several
    runs (its weights are shared, each run has a cache of its own).
    ``cache_of`` names an earlier run whose cache this run reads instead of
    writing one of its own.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartSpec
    final_norm: PartSpec
    lm_head: PartSpec
    positions: Dict[str, PartSpec]
    layers: List[LayerSpec]
    schedule: List[Run]

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.schedule:
            raise ValueError("a model needs a non-empty schedule")
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule[{i}] names layer {run.layer}, "
                                 f"but there are {len(self.layers)} layers")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < i:
                    raise ValueError(
                        f"schedule[{i}] reads the cache of run {run.cache_of}, "
                        "which is not an earlier run")
                if self.schedule[run.cache_of].cache_of is not None:
                    raise ValueError(
                        f"schedule[{i}] reads the cache of run {run.cache_of}, "
                        "which has no cache of its own")
            layer = self.layers[run.layer]
            if layer.position is not None and layer.position not in self.positions:
                raise ValueError(f"layer {run.layer} uses position encoding "
                                 f"'{layer.position}', which the spec does not define")
