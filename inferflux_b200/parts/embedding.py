"""Token embedding and output head.

Embedding: ``residual[t, :] = float32(E[id_t, :])``, no scale (reference:
runtime/backends/cuda/native/cuda_kernels.cu:599-614).  Output head:
``logits = x W^T`` with ``W = lm_head.weight [V, H]`` or the embedding table
when the head is tied (reference falls back to the embedding when
``lm_head.weight`` is absent, runtime/backends/cuda/native/weight_map.cpp:33-37);
logits come out in float32 (the reference rounds them to 16 bits first,
transformer_forward.cu:2178-2189).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import IGNORED, MATRIX, WeightSpec
from .base import Part
from .linear import Linear


class TokenEmbedding(Part):
    """params: ``vocab``, ``hidden``, ``name`` (weight ``<name>.weight``)."""

    family = "embedding"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.vocab, self.hidden = int(params["vocab"]), int(params["hidden"])
        self.table: torch.Tensor = None

    @classmethod
    def weight_specs(cls, params, prefix) -> List[WeightSpec]:
        return [WeightSpec(cls.full_name(prefix, params, "weight"), (int(params["vocab"]), int(params["hidden"])), MATRIX)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.full_name(self.prefix, self.params, "weight")].contiguous()

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        out = torch.empty((token_ids.numel(), self.hidden), dtype=torch.float32, device=token_ids.device)
        return ops.embed_gather(self.table, token_ids, out)


class LinearHead(Part):
    """params: ``vocab``, ``hidden``, ``name``, ``tied_to`` (None, or the full
    name of the embedding table to use instead of a weight of its own)."""

    family = "lm_head"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.vocab, self.hidden = int(params["vocab"]), int(params["hidden"])
        self.linear: Linear = None

    @classmethod
    def weight_specs(cls, params, prefix) -> List[WeightSpec]:
        shape = (int(params["vocab"]), int(params["hidden"]))
        name = cls.full_name(prefix, params, "weight")
        if params.get("tied_to"):
            return [WeightSpec(name, shape, IGNORED, optional=True)]
        return [WeightSpec(name, shape, MATRIX)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        src = self.params.get("tied_to") or self.full_name(self.prefix, self.params, "weight")
        self.linear = Linear(tensors[src])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [W, hidden] -> float32 logits [W, vocab]."""
        return self.linear.forward(x, out_dtype=torch.float32)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("lm_head", "linear_head", LinearHead)
