"""Feed-forward parts.

``swiglu``: ``down( silu(gate(x)) * up(x) )`` with ``silu(g) = g / (1 + exp(-g))``
in float32, no biases (reference:
runtime/backends/cuda/native/transformer_forward.cu:1877-1879,1912-1914 gate
and up, :1981-1983 activation, :2024-2026 down;
runtime/backends/cuda/native/cuda_kernels.cu:137-149).  The reference runs
gate and up as two products and the activation as a kernel of its own; here
their weights are stacked at load and in bfloat16 one kernel does the product
and the activation, so the ``[gate | up]`` intermediate never goes to memory:
the weight-streaming kernel for a few rows, the tcgen05 product for many.
"""
from __future__ import annotations

from typing import Any, Dict, List

import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import MATRIX, WeightSpec
from .base import Part
from .linear import Linear


FUSED_PRODUCT_ROWS = 128   # above this many rows gate/up + activation run as one tcgen05 product (measured: 256 rows 63 us
                           # against 76 us for library product + activation kernel; at 64 rows the library is ahead)


class SwiGLU(Part):
    """params: ``hidden``, ``intermediate``, ``name`` (weights are
    ``<prefix>.<name>.{gate,up,down}_proj.weight``)."""

    family = "feed_forward"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden"])
        self.intermediate = int(params["intermediate"])
        self.gate_up: Linear = None
        self.down: Linear = None

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, i = int(params["hidden"]), int(params["intermediate"])
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        return [WeightSpec(n("gate_proj.weight"), (i, h), MATRIX),
                WeightSpec(n("up_proj.weight"), (i, h), MATRIX),
                WeightSpec(n("down_proj.weight"), (h, i), MATRIX)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        gate, up = tensors.pop(n("gate_proj.weight")), tensors.pop(n("up_proj.weight"))
        if gate.dtype != up.dtype:
            gate, up = gate.float(), up.float()
        self.gate_up = Linear(torch.cat([gate, up], dim=0))
        del gate, up
        self.down = Linear(tensors.pop(n("down_proj.weight")))

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        w = self.gate_up.weight
        act = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
        fused = w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and self.hidden % 8 == 0
        if fused and x.shape[0] <= ops.GEMV_MAX_ROWS:         # (up to 16 rows the fused kernel beats library product + activation)
            ops.gemv_bf16(x, w, None, act, swiglu=True)       # product and activation in one kernel
        elif fused and x.is_contiguous() and x.shape[0] > FUSED_PRODUCT_ROWS:
            ops.gemm_umma(x, w, None, act, swiglu=True)       # many rows: tcgen05 product, activation in its epilogue
        else:
            ops.swiglu(self.gate_up.forward(x), act)
        return self.down.forward(act, out_dtype=x.dtype, allow_partials=True)


register_part("feed_forward", "swiglu", SwiGLU)
