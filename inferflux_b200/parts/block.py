"""How a layer's parts are arranged.

``prenorm`` (the reference's only block,
runtime/backends/cuda/native/transformer_forward.cu:1400-2103):

    x  = norm_1(residual)          residual is the float32 stream
    residual += mixer(x)
    x2 = norm_2(residual)
    residual += feed_forward(x2)

The second sum is not done here: the block returns the feed-forward's output
as a pending delta, and the next block's first norm (or the final norm) adds
it in the same kernel that norms (the reference fuses the same pair,
transformer_forward.cu:2054-2077).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.registry import register_part
from .base import RunInfo


class PreNormBlock:
    """An arrangement declares its roles (role -> family of the part that fills
    it) and is built from the layer's parts by role; ``optional_roles`` may be
    left out of a layer."""

    family = "arrangement"
    roles = {"mixer": "mixer", "mixer_norm": "norm", "feed_forward": "feed_forward", "feed_forward_norm": "norm"}
    optional_roles = frozenset()

    def __init__(self, parts: Dict[str, object], position_name: Optional[str]):
        self.mixer = parts["mixer"]
        self.mixer_norm = parts["mixer_norm"]
        self.feed_forward = parts["feed_forward"]
        self.feed_forward_norm = parts["feed_forward_norm"]
        self.position_name = position_name

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx, run: RunInfo) -> torch.Tensor:
        """residual float32 [N, H] (updated in place); delta = the previous
        block's pending output or None.  Returns this block's pending output."""
        x = self.mixer_norm.forward(residual, delta)
        position = ctx.position_tables.get(self.position_name) if self.position_name else None
        a = self.mixer.forward(x, ctx, run, position)
        x2 = self.feed_forward_norm.forward(residual, a)
        return self.feed_forward.forward(x2, ctx)


register_part("arrangement", "prenorm", PreNormBlock)
