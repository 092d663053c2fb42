"""Mixers.  ``gqa_attention``: causal grouped-query attention over the paged
cache.

Per token (reference, in this order):
  q, k, v = x Wq^T, x Wk^T, x Wv^T      runtime/backends/cuda/native/transformer_forward.cu:1479-1481,1514-1517,1550-1553
  += biases (those that exist)          :1567-1608, runtime/backends/cuda/native/cuda_kernels.cu:694-723
  rotate q and k by the token position  :1632-1634
  k, v -> cache                         :1652-1653
  head h attends with kv head h / (n_heads / n_kv); s = (q . k) / sqrt(d) after
  the dot; causal; float32 online softmax
                                        runtime/backends/cuda/kernels/flash_attention.cu:52-173
  o = attn Wo^T (no bias in Qwen2)      transformer_forward.cu:1719-1727
The reference keeps q, k, v as three products and a separate bias kernel;
here the three weights are stacked at load, and one kernel adds the bias,
rotates and writes the cache.  ``window`` (None = all keys) hides keys more
than ``window - 1`` positions behind the query; the reference has no window.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, WeightSpec
from .base import KVNeed, Part, PartialSums, RunInfo
from .linear import Linear


class GQAttention(Part):
    """params: ``hidden``, ``n_heads``, ``n_kv_heads``, ``head_dim``,
    ``qkv_bias``, ``o_bias``, ``window`` (None or int), ``kv_shared`` (True: the
    layer has only q and o and reads another run's cache), ``scale`` (None =
    ``1/sqrt(head_dim)``), ``name``."""

    family = "mixer"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        p = params
        self.hidden = int(p["hidden"])
        self.n_heads, self.n_kv, self.head_dim = int(p["n_heads"]), int(p["n_kv_heads"]), int(p["head_dim"])
        self.window = int(p["window"]) if p.get("window") else 0
        self.kv_shared = bool(p.get("kv_shared", False))
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        if self.n_heads % self.n_kv:
            raise ValueError(f"n_heads {self.n_heads} is not a multiple of n_kv_heads {self.n_kv}")
        if self.head_dim % 2 or not 2 <= self.head_dim <= 256:
            raise ValueError(f"head_dim {self.head_dim} must be even and within 2..256")
        self.qkv: Linear = None
        self.qkv_bias: Optional[torch.Tensor] = None
        self.o: Linear = None

    # -- declarations ----------------------------------------------------
    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, nh, nkv, hd = (int(params[k]) for k in ("hidden", "n_heads", "n_kv_heads", "head_dim"))
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        shared = bool(params.get("kv_shared", False))
        specs = [WeightSpec(n("q_proj.weight"), (nh * hd, h), MATRIX)]
        if not shared:
            specs += [WeightSpec(n("k_proj.weight"), (nkv * hd, h), MATRIX),
                      WeightSpec(n("v_proj.weight"), (nkv * hd, h), MATRIX)]
        if params.get("qkv_bias"):
            specs.append(WeightSpec(n("q_proj.bias"), (nh * hd,), VECTOR))
            if not shared:
                specs += [WeightSpec(n("k_proj.bias"), (nkv * hd,), VECTOR),
                          WeightSpec(n("v_proj.bias"), (nkv * hd,), VECTOR)]
        specs.append(WeightSpec(n("o_proj.weight"), (h, nh * hd), MATRIX))
        if params.get("o_bias"):
            specs.append(WeightSpec(n("o_proj.bias"), (h,), VECTOR))
        return specs

    @classmethod
    def kv_need(cls, params: Dict[str, Any]) -> Optional[KVNeed]:
        if params.get("kv_shared"):
            return None
        return KVNeed(int(params["n_kv_heads"]), int(params["head_dim"]),
                      int(params["window"]) if params.get("window") else None)

    # -- weights ---------------------------------------------------------
    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        names = ["q_proj"] if self.kv_shared else ["q_proj", "k_proj", "v_proj"]
        mats = [tensors.pop(n(f"{x}.weight")) for x in names]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.qkv = Linear(torch.cat(mats, dim=0) if len(mats) > 1 else mats[0])
        del mats
        if self.params.get("qkv_bias"):
            self.qkv_bias = torch.cat([tensors.pop(n(f"{x}.bias")).float() for x in names]).contiguous()
        o_bias = tensors.pop(n("o_proj.bias")) if self.params.get("o_bias") else None
        self.o = Linear(tensors.pop(n("o_proj.weight")), o_bias)

    # -- the step --------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx, run: RunInfo, position) -> torch.Tensor:
        """x [N, hidden] (normed) -> [N, hidden]; writes this step's keys and
        values into the run's cache (unless it reads another run's) and
        attends over the cache."""
        n = x.shape[0]
        nkv_w = 0 if self.kv_shared else self.n_kv
        if position is not None:
            cos, sin = position
        else:
            cos = sin = torch.empty((n, 0), dtype=torch.float32, device=x.device)
        # a few rows: the product may come as float32 partial sums, which the kernel below adds up
        partials = None
        qkv = self.qkv.forward(x, allow_partials=2 * cos.shape[1] == self.head_dim and self.head_dim % 16 == 0)
        if isinstance(qkv, PartialSums):
            partials = qkv.tensor
            qkv = torch.empty(partials.shape[1:], dtype=x.dtype, device=x.device)
        g = run.kv_group
        k_layer, v_layer, page_stride = ctx.kv.layer_views(g, run.kv_index)
        attn = torch.empty((n, self.n_heads * self.head_dim), dtype=qkv.dtype, device=x.device)
        if (ctx.n_decode == n and not ctx.n_chunk_tiles and nkv_w and qkv.dtype == torch.bfloat16
                and self.head_dim in ops.FAST_ATTENTION_HEAD_DIMS and 2 * cos.shape[1] == self.head_dim
                and not self._share_by_tiles(ctx)):
            # single tokens only: the attention kernel adds the bias, rotates and writes the cache itself
            self.decode(qkv, attn, ctx, g, k_layer, v_layer, page_stride,
                        prep=(self.qkv_bias, cos, sin, ctx.slot_maps[g], partials))
            return self.o.forward(attn, out_dtype=x.dtype, allow_partials=True)
        ops.qkv_rope_kv_write(qkv, self.qkv_bias, cos, sin, ctx.slot_maps[g] if nkv_w else None,
                              k_layer if nkv_w else None, v_layer if nkv_w else None, page_stride,
                              ctx.page_size, self.n_heads, nkv_w, self.head_dim, partials)
        self.attend(qkv, attn, ctx, g, k_layer, v_layer, page_stride)
        return self.o.forward(attn, out_dtype=x.dtype, allow_partials=True)

    def attend(self, qkv, attn, ctx, g, k_layer, v_layer, page_stride) -> None:
        """bfloat16 with a head size the tensor-core kernels take: prompt
        portions go to the tcgen05 kernel (head size 128) or the mma.sync kernel
        (64), single tokens to the split decode kernel; anything else (float32,
        other head sizes) to the generic kernel."""
        common = (ctx.entry_q_start, ctx.entry_q_len, ctx.entry_ctx_start)
        if qkv.dtype != torch.bfloat16 or self.head_dim not in ops.FAST_ATTENTION_HEAD_DIMS:
            ops.attn_paged_generic(qkv, qkv.stride(0), attn, k_layer, v_layer, page_stride, ctx.page_size,
                                   ctx.block_tables[g], ctx.tile_entry, ctx.tile_q0, ctx.n_tiles, *common,
                                   self.n_heads, self.n_kv, self.head_dim, self.scale, self.window)
            return
        if ctx.n_chunk_tiles and self.head_dim == ops.UMMA_ATTENTION_HEAD_DIM:
            max_keys = min(ctx.max_ctx_len, self.window + 128) if self.window else ctx.max_ctx_len
            splits = ops.attn_prefill_umma_splits(ctx.n_umma_tiles, self.n_heads, max_keys)
            ops.attn_prefill_umma(qkv, qkv.stride(0), attn, k_layer, v_layer, page_stride, ctx.page_size,
                                  ctx.block_tables[g], ctx.umma_tile_entry, ctx.umma_tile_q0, ctx.n_umma_tiles,
                                  *common, self.n_heads, self.n_kv, self.head_dim, self.scale, self.window, splits)
        elif ctx.n_chunk_tiles:
            ops.attn_prefill_bf16(qkv, qkv.stride(0), attn, k_layer, v_layer, page_stride, ctx.page_size,
                                  ctx.block_tables[g], ctx.chunk_tile_entry, ctx.chunk_tile_q0, ctx.n_chunk_tiles,
                                  *common, self.n_heads, self.n_kv, self.head_dim, self.scale, self.window)
        if ctx.n_decode:
            self.decode(qkv, attn, ctx, g, k_layer, v_layer, page_stride)

    def _share_by_tiles(self, ctx) -> bool:
        """Contexts of very different lengths (and no window that evens them
        out): the kernel that shares the tiles of all entries out evenly."""
        return (ctx.decode_skewed and ctx.n_decode <= ops.DECODE_EVEN_MAX_ENTRIES
                and not (self.window and self.window < 1024))

    def decode(self, qkv, attn, ctx, g, k_layer, v_layer, page_stride, prep=None) -> None:
        """The step's single tokens.  Contexts of about the same length: the keys
        of each are cut into as many parts as fill the GPU, and merged; with
        ``prep`` = (bias, cos, sin, slot map, partial sums or None) qkv is
        still the bare product and the kernel prepares q, k and v itself.
        Contexts of very different lengths: all their tiles are shared out
        evenly over the blocks."""
        max_keys = min(ctx.max_ctx_len, self.window) if self.window else ctx.max_ctx_len
        if prep is None and self._share_by_tiles(ctx):
            pieces = ops.attn_decode_pieces(self.n_heads, self.n_kv, self.head_dim, max_keys)
            rows = ctx.n_decode * self.n_heads * pieces
            part_o = torch.empty(rows * self.head_dim, dtype=torch.float32, device=qkv.device)
            part_ml = torch.empty(rows * 2, dtype=torch.float32, device=qkv.device)
            count = torch.empty(ctx.n_decode * self.n_heads, dtype=torch.int32, device=qkv.device)
            ops.attn_decode_even_bf16(qkv, attn, k_layer, v_layer, page_stride, ctx.page_size, ctx.block_tables[g],
                                      ctx.decode_entries, ctx.n_decode, ctx.entry_q_start, ctx.entry_q_len,
                                      ctx.entry_ctx_start, part_o, part_ml, count, self.n_heads, self.n_kv, self.head_dim,
                                      self.scale, self.window, pieces)
            return
        n_splits = ops.attn_decode_splits(ctx.n_decode, self.n_heads, self.n_kv, self.head_dim, max_keys)
        part_o = part_ml = None
        if n_splits > 1:
            rows = ctx.n_decode * self.n_heads * n_splits
            part_o = torch.empty(rows * self.head_dim, dtype=torch.float32, device=qkv.device)
            part_ml = torch.empty(rows * 2, dtype=torch.float32, device=qkv.device)
        meta = (k_layer, v_layer, page_stride, ctx.page_size, ctx.block_tables[g], ctx.decode_entries, ctx.n_decode,
                ctx.entry_q_start, ctx.entry_q_len, ctx.entry_ctx_start, part_o, part_ml,
                self.n_heads, self.n_kv, self.head_dim, self.scale, self.window, n_splits)
        if prep is None:
            ops.attn_decode_bf16(qkv, qkv.stride(0), attn, *meta)
        else:
            bias, cos, sin, slot_map, partials = prep
            ops.attn_decode_prep_bf16(qkv, bias, cos, sin, slot_map, partials, attn, *meta)


register_part("mixer", "gqa_attention", GQAttention)
