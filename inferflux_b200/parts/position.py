"""Position encodings.  A position part turns a step's token positions into
whatever its mixers need, once per step for all layers that share it.

``rotary_half``: rotate-half rotary positions.  For ``i`` in ``[0, d/2)``:
``f_i = theta^(-2i/d)``, ``a = pos * f_i``, and the pair ``(x_i, x_{i+d/2})``
is rotated by ``a`` (reference: runtime/backends/cuda/native/cuda_kernels.cu:70-115,
rope_type 2, selected for ``qwen2`` at
runtime/backends/cuda/native/model_loader.h:45-58).  The reference evaluates
``powf/cosf/sinf`` per element, per layer; here the cos/sin tables are made
once per step in double precision and rounded to float32.
"""
from __future__ import annotations


import torch

from ..config.registry import register_part
from ..kernels import ops
from .base import Part


class RotaryHalf(Part):
    """params: ``rotary_dim`` (how many leading dims of a head rotate),
    ``theta``."""

    family = "position"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.rotary_dim = int(params["rotary_dim"])
        self.theta = float(params["theta"])
        if self.rotary_dim % 2 or self.rotary_dim < 0:
            raise ValueError(f"rotary_dim must be even and >= 0, got {self.rotary_dim}")
        half = self.rotary_dim // 2
        i = torch.arange(half, dtype=torch.float64)
        self.inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                                  -2.0 * i / max(self.rotary_dim, 1)).to(device)

    def prepare(self, ctx) -> None:
        """Make ``(cos, sin)`` float32 ``[N, rotary_dim/2]`` for the step's positions."""
        half = self.rotary_dim // 2
        cos = torch.empty((ctx.n_tokens, half), dtype=torch.float32, device=ctx.device)
        sin = torch.empty((ctx.n_tokens, half), dtype=torch.float32, device=ctx.device)
        if half:
            ops.rope_table(ctx.positions, self.inv_freq, cos, sin)
        return cos, sin


register_part("position", "rotary_half", RotaryHalf)
