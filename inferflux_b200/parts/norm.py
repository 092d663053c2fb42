"""Root-mean-square norm fused with the residual sum.

``residual += delta;  out = residual * rsqrt(mean(residual^2) + eps) * weight``
in float32 on the float32 residual stream, rounded once on output
(reference: runtime/backends/cuda/native/cuda_kernels.cu:469-501 norm,
:541-579 fused add + norm; call sites
runtime/backends/cuda/native/transformer_forward.cu:1413-1424,1744-1754).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import VECTOR, WeightSpec
from .base import Part, PartialSums


class RMSNorm(Part):
    """params: ``hidden``, ``eps``, ``name`` (weight is ``<prefix>.<name>.weight``)."""

    family = "norm"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden"])
        self.eps = float(params["eps"])
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        return [WeightSpec(cls.full_name(prefix, params, "weight"), (int(params["hidden"]),), VECTOR,
                           init="one_plus_normal")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.full_name(self.prefix, self.params, "weight")].to(torch.float32).contiguous()

    def forward(self, residual: torch.Tensor, delta, out: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Adds ``delta`` (a tensor, a :class:`PartialSums` or None) into the
        float32 ``residual`` (unless ``rows`` picks rows, which leaves it
        untouched) and returns the normed rows in the engine's type."""
        n_partials = 1
        if isinstance(delta, PartialSums):
            delta, n_partials = delta.tensor, delta.count
        n_rows = rows.numel() if rows is not None else residual.shape[0]
        if out is None:
            out = torch.empty((n_rows, self.hidden), dtype=self.dtype, device=residual.device)
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows, n_partials)


register_part("norm", "rmsnorm", RMSNorm)
