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
class CacheStream:
    """One tensor that a mixer keeps per token in the paged cache: ``heads``
    vectors of ``width`` elements.  Within a page a stream lies as
    ``[head][slot][width]``, so one head's vectors of a page are contiguous."""

    name: str
    heads: int
    width: int


@dataclass(frozen=True)
class KVNeed:
    """What a mixer keeps per token in pages: one or more streams (keys and
    values for attention; a single latent vector for a mixer that caches
    one), and for how long: ``window`` None = every token is kept, w = only
    the last w.  Runs whose mixers ask for equal needs share a cache group."""

    streams: Tuple[CacheStream, ...]
    window: Optional[int] = None

    @classmethod
    def keys_and_values(cls, n_kv_heads: int, head_dim: int, window: Optional[int] = None) -> "KVNeed":
        """``n_kv_heads * head_dim`` keys and as many values per token."""
        return cls((CacheStream("k", n_kv_heads, head_dim), CacheStream("v", n_kv_heads, head_dim)), window)

    @property
    def elements_per_token(self) -> int:
        return sum(s.heads * s.width for s in self.streams)


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
    the weight-name prefix of the enclosing layer ("" at model level).

    Interfaces by family (``x`` = ``[N, hidden]`` rows of the step's flattened
    tokens, ``ctx`` = the step's :class:`~inferflux_b200.engine.batch.StepContext`):

    * ``mixer``: ``forward(x, ctx, run, position) -> Tensor | PartialSums``.
      ``run`` is the :class:`RunInfo` of this execution of the layer (its cache
      group and index, its state tensors); ``position`` is whatever the position
      encoding named by the layer returned from ``prepare`` for this step, or
      None.
    * ``feed_forward``: ``forward(x, ctx) -> Tensor | PartialSums``.
    * ``norm``: ``forward(residual, delta, out=None, rows=None) -> Tensor``:
      adds ``delta`` (tensor, PartialSums or None) into the float32 residual
      unless ``rows`` selects rows, returns the normed rows.
    * ``position``: ``prepare(ctx) -> object``, once per step for all layers.
      The contract between a position encoding and the mixers that consume it
      is the type of that object.  The built-in ``gqa_attention`` takes a pair
      ``(cos, sin)`` of float32 ``[N, r/2]`` tensors, ``r <= head_dim`` even,
      and rotates the first ``r`` dimensions of every query and key head in
      split-half pairs ``(i, i + r/2)``; any position part that returns such a
      pair serves it.  A mixer with another idea of position defines its own
      object and says so in its docstring.
    * ``embedding``: ``forward(token_ids) -> float32 [N, hidden]``;
      ``lm_head``: ``forward(x) -> float32 [rows, vocab]``.

    Any part may describe the step for its kernels (:meth:`describe_step`).
    """

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

    # -- the step -------------------------------------------------------
    #: Parts with the same key share one description per step (the key names the
    #: kind of description, e.g. the tile lists of one family of kernels); None =
    #: the part needs none.
    describe_key: Optional[str] = None

    def describe_step(self, layout, put) -> object:
        """Per-step metadata for this part's kernels, derived on the host from
        ``layout`` (:class:`~inferflux_b200.engine.batch.StepLayout`: how many
        tokens each entry brings and how many it has cached).  ``put(values)``
        appends int32 values to the step's metadata (one host-to-device copy for
        the whole step) and returns their device view.  The result is kept in
        ``ctx.extras[describe_key]``.  Called once per step and key, before the
        copy; in a captured step of single tokens the copy is repeated with new
        token ids, positions and block tables only, so what this writes for such
        a step may depend on the number of entries and on :meth:`step_shape`
        alone."""
        return None

    def step_shape(self, layout) -> tuple:
        """What, beyond the number of entries and the width of the block tables,
        decides which kernels this part launches in a step of single tokens (it
        becomes part of the key under which such steps are captured)."""
        return ()


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
