"""A matrix product ``y = x W^T (+ b)`` with ``W`` stored ``[out, in]``.

The reference issues one cuBLAS call per projection with float32 accumulation
(runtime/backends/cuda/native/cublas_gemm.cpp:84-102, ``C[M,N] = A[M,K] *
B[N,K]^T``).  Here a float32 weight goes through the FFMA kernel of the 32-bit
path; a bfloat16 weight goes through the library (cuBLAS via ``torch.mm``) for
many rows, through the weight-streaming kernel (gemv_bf16.cu) for up to 8
rows, and through the tcgen05 kernel with the operands' places changed
(gemm_umma.cu) for up to 128 rows against a long K.  This is not a registered part: mixers and feed-forwards own their
Linears.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import PartialSums


GEMV_ROWS = 8     # up to this many rows go to the weight-streaming kernel (it matches the library there)
# From 9 to 128 rows a product is still bound by reading W once.  The tcgen05 kernel with the weights as the
# tiles' rows beats the library there by a tenth when K is long (the down projection: 27 against 31 us at 64
# rows); with a short K its set-up weighs more than it saves (qkv, o: 10 against 9 us), so those stay.
FEW_ROWS, FEW_ROWS_MIN_K = 128, 8192


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        if weight.dim() != 2:
            raise ValueError("Linear wants a [out, in] matrix")
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape
        self.bias = None if bias is None else bias.to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None, allow_partials: bool = False,
                f32_sums: bool = False):
        """x [M, in] -> [M, out] in ``out_dtype`` (default: x's type).  With
        ``allow_partials`` the result may be a :class:`PartialSums` (the
        weight-streaming kernel cuts K between blocks when a matrix has too few
        rows to fill the GPU).  With ``f32_sums`` on top of that, a bfloat16
        product always comes as float32 sums (one slice from the library): for
        a consumer that computes on with the sums, to which a rounding to
        bfloat16 in between would only add error."""
        m = x.shape[0]
        out_dtype = out_dtype or x.dtype
        w = self.weight
        if w.dtype == torch.float32:
            # 32-bit weights: true float32 product whatever the activations are
            if x.dtype != torch.float32:
                x = ops.convert(x.contiguous(), torch.empty(x.shape, dtype=torch.float32, device=x.device))
            y = torch.empty((m, self.out_features), dtype=torch.float32, device=x.device)
            ops.gemm_f32(x, w, self.bias, y)
            if out_dtype != torch.float32:
                y = ops.convert(y, torch.empty(y.shape, dtype=out_dtype, device=x.device))
            return y
        if x.dtype != torch.bfloat16:
            raise ops.KernelError(f"Linear: bfloat16 weights need bfloat16 activations, got {x.dtype}")
        if m <= GEMV_ROWS and self.in_features % 8 == 0:
            # a few rows: bound by reading the weights once -> the weight-streaming kernel
            splits = self._k_splits() if allow_partials else 1
            if splits > 1:
                y = torch.empty((splits, m, self.out_features), dtype=torch.float32, device=x.device)
                return PartialSums(ops.gemv_bf16(x, w, self.bias, y, k_splits=splits))
            if allow_partials and f32_sums:
                y = torch.empty((m, self.out_features), dtype=torch.float32, device=x.device)
                return PartialSums(ops.gemv_bf16(x, w, self.bias, y).unsqueeze(0))
            y = torch.empty((m, self.out_features), dtype=out_dtype, device=x.device)
            return ops.gemv_bf16(x, w, self.bias, y)
        if (allow_partials and self.bias is None and m <= FEW_ROWS and self.in_features >= FEW_ROWS_MIN_K
                and self.in_features % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0):
            parts = ops.gemm_umma_skinny_parts(self.out_features, self.in_features)
            y = torch.empty((parts, m, self.out_features), dtype=torch.float32, device=x.device)
            return PartialSums(ops.gemm_umma_skinny(x, w, y))
        if allow_partials and f32_sums and self.bias is None:
            return PartialSums(ops.matmul_library(x, w, torch.float32).unsqueeze(0))
        y = ops.matmul_library(x, w, torch.float32 if (out_dtype == torch.float32 or self.bias is not None)
                               else torch.bfloat16)
        if self.bias is not None:
            y += self.bias
        return y if y.dtype == out_dtype else y.to(out_dtype)

    def _k_splits(self) -> int:
        """Into how many parts the weight-streaming kernel cuts K (it knows its
        block shapes and how many blocks the GPU holds; the number depends on
        the matrix only, never on the batch)."""
        return ops.gemv_k_splits(self.out_features, self.in_features)
