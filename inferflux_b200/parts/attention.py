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
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, WeightSpec
from .base import KVNeed, Part, PartialSums, RunInfo
from .linear import Linear


QUERY_TILE = 16     # tokens per query tile of the generic attention kernel
CHUNK_TILE = 64     # tokens per query tile of the mma.sync kernel for prompt portions
FUSED_QKV_MIN_ROWS = 2048   # from this many rows on q, k, v may come from the product with the fused epilogue
UMMA_TILE = ops.UMMA_ATTENTION_TILE   # tokens per query tile of the tcgen05 kernel for prompt portions (256)


def contexts_skewed(lengths) -> bool:
    """Whether the contexts of a step's single tokens differ so much in length
    that attention should share its work out by tiles and not by requests: the
    longest is at least 1,024 tokens and at least 1.5 times the mean.  With
    equal contexts the kernel that gives every request its own blocks is about
    a fifth faster; with one long context among short ones it takes as long as
    the long one alone."""
    n = len(lengths)
    if n < 2:
        return False
    longest = max(lengths)
    return longest >= 1024 and 2 * longest * n >= 3 * sum(lengths)


@dataclass
class AttentionStep:
    """What the attention kernels read of a step beyond the common metadata: the
    step's query tiles at the three tile sizes of the kernels, and which entries
    bring a single token.  int32 device tensors with their lengths."""

    tile_entry: torch.Tensor                  # [T] query tiles of QUERY_TILE tokens (all entries)
    tile_q0: torch.Tensor                     # [T] first query of the tile within its entry
    n_tiles: int
    chunk_tile_entry: torch.Tensor            # [Tc] tiles of CHUNK_TILE tokens over entries with more than one token
    chunk_tile_q0: torch.Tensor
    n_chunk_tiles: int
    umma_tile_entry: torch.Tensor             # [Tu] tiles of umma_tile_rows tokens over the same entries
    umma_tile_q0: torch.Tensor
    n_umma_tiles: int
    umma_tile_rows: int                       # UMMA_TILE, or half of it where tiles that high would leave SMs idle
    decode_entries: torch.Tensor              # [D] entries that bring exactly one token
    n_decode: int
    decode_skewed: bool                       # their contexts differ much in length (contexts_skewed)


class GQAttention(Part):
    """params: ``hidden``, ``n_heads``, ``n_kv_heads``, ``head_dim``,
    ``qkv_bias``, ``o_bias``, ``window`` (None or int), ``kv_shared`` (True: the
    layer has only q and o and reads another run's cache), ``scale`` (None =
    ``1/sqrt(head_dim)``), ``name``.

    Position: a pair ``(cos, sin)`` of float32 ``[N, r/2]`` tensors (``r`` even,
    at most ``head_dim``): the first ``r`` dimensions of every query and key
    head are rotated in split-half pairs ``(i, i + r/2)``; None = no rotation."""

    family = "mixer"
    describe_key = "gqa_attention"

    # -- the step's description, once for all attention layers ------------
    def describe_step(self, layout, put) -> AttentionStep:
        tile_entry, tile_q0, ctile_entry, ctile_q0, utile_entry, utile_q0, dec = [], [], [], [], [], [], []
        # The tcgen05 kernel gives a block (an SM) to a tile and head.  Tiles of 256 tokens share their key tiles
        # between two query tiles; where they would take half the SMs or fewer, tiles of 128 make twice the
        # blocks (measured, 7B shapes: 512 tokens at 2,048 of context 26.6 against 37.4 us, 512 alone 11.7 / 14.6;
        # at 768 and 1,024 tokens, 84 and 112 blocks of 256, the higher tiles win by up to a tenth).
        portions = [int(n) for n in layout.q_len[:layout.n_entries] if int(n) > 1]
        blocks = sum((n + UMMA_TILE - 1) // UMMA_TILE for n in portions) * self.n_heads
        on_gpu = torch.device(self.device).type == "cuda"
        utile = UMMA_TILE // 2 if portions and on_gpu and 2 * blocks <= ops.sm_count(self.device) else UMMA_TILE
        for i in range(layout.n_entries):
            ln = int(layout.q_len[i])
            if ln == 1:
                tile_entry.append(i), tile_q0.append(0), dec.append(i)
                continue
            for q0 in range(0, ln, QUERY_TILE):
                tile_entry.append(i), tile_q0.append(q0)
            for q0 in range(0, ln, CHUNK_TILE):
                ctile_entry.append(i), ctile_q0.append(q0)
            for q0 in range(0, ln, utile):
                utile_entry.append(i), utile_q0.append(q0)
        return AttentionStep(
            put(tile_entry), put(tile_q0), len(tile_entry), put(ctile_entry), put(ctile_q0), len(ctile_entry),
            put(utile_entry), put(utile_q0), len(utile_entry), utile, put(dec), len(dec),
            contexts_skewed([int(layout.ctx_start[i]) + 1 for i in dec]))

    def step_shape(self, layout) -> tuple:
        """The kernel for single tokens is chosen by how much the contexts differ."""
        return (contexts_skewed([int(c) + 1 for c, n in zip(layout.ctx_start, layout.q_len) if n == 1]),)

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
        return KVNeed.keys_and_values(int(params["n_kv_heads"]), int(params["head_dim"]),
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
        step: AttentionStep = ctx.extras[self.describe_key]
        if position is not None:
            if not (isinstance(position, (tuple, list)) and len(position) == 2):
                raise TypeError("gqa_attention takes its position as a pair (cos, sin) of [N, r/2] float32 tensors; "
                                f"the layer's position encoding gave {type(position).__name__}")
            cos, sin = position
        else:
            cos = sin = torch.empty((n, 0), dtype=torch.float32, device=x.device)
        g = run.kv_group
        k_layer, v_layer, page_stride = ctx.kv.layer_views(g, run.kv_index)
        if self._fused_qkv(x, n, cos):
            # many rows: one kernel makes the product, adds the bias, rotates and writes the cache
            q = torch.empty((n, self.n_heads * self.head_dim), dtype=x.dtype, device=x.device)
            ops.gemm_umma_qkv(x, self.qkv.weight, self.qkv_bias, q, cos, sin, ctx.slot_maps[g] if nkv_w else None,
                              k_layer if nkv_w else None, v_layer if nkv_w else None, page_stride, ctx.page_size,
                              self.n_heads, nkv_w)
            attn = torch.empty_like(q)
            self.attend(q, attn, ctx, step, g, k_layer, v_layer, page_stride)
            return self.o.forward(attn, out_dtype=x.dtype, allow_partials=True)
        # a few rows: the product may come as float32 partial sums, which the kernel below adds up
        partials = None
        # (q and k go on into the rotation and the scores: their product is taken as float32 sums wherever the
        # kernel below can add such up; rounded to bfloat16 first, the logits behind 2,048 tokens were off by
        # 2 % of the largest instead of 1.2 %)
        sums = 2 * cos.shape[1] == self.head_dim and self.head_dim % 16 == 0
        qkv = self.qkv.forward(x, allow_partials=sums, f32_sums=sums)
        if isinstance(qkv, PartialSums):
            partials = qkv.tensor
            qkv = torch.empty(partials.shape[1:], dtype=x.dtype, device=x.device)
        attn = torch.empty((n, self.n_heads * self.head_dim), dtype=qkv.dtype, device=x.device)
        if (step.n_decode == n and not step.n_chunk_tiles and nkv_w and qkv.dtype == torch.bfloat16
                and self.head_dim in ops.FAST_ATTENTION_HEAD_DIMS and 2 * cos.shape[1] == self.head_dim
                and not self._share_by_tiles(step)):
            # single tokens only: the attention kernel adds the bias, rotates and writes the cache itself
            self.decode(qkv, attn, ctx, step, g, k_layer, v_layer, page_stride,
                        prep=(self.qkv_bias, cos, sin, ctx.slot_maps[g], partials))
            return self.o.forward(attn, out_dtype=x.dtype, allow_partials=True)
        ops.qkv_rope_kv_write(qkv, self.qkv_bias, cos, sin, ctx.slot_maps[g] if nkv_w else None,
                              k_layer if nkv_w else None, v_layer if nkv_w else None, page_stride,
                              ctx.page_size, self.n_heads, nkv_w, self.head_dim, partials)
        self.attend(qkv, attn, ctx, step, g, k_layer, v_layer, page_stride)
        return self.o.forward(attn, out_dtype=x.dtype, allow_partials=True)

    def _fused_qkv(self, x: torch.Tensor, n: int, cos: torch.Tensor) -> bool:
        """Whether the step's q, k, v come from the tcgen05 product with bias,
        rotation and cache write in its epilogue: bfloat16, head size 128
        rotated as a whole, and rows enough that it beats the library product
        followed by the separate kernel.  It does when its tiles of 256 x 256
        fill the rounds that the pairs of SMs make over them (measured, us,
        fused against separate: 7B sizes 2,048 rows 49.7 / 58.0, 2,560 rows
        67.3 / 78.5, 4,096 rows 91 / 106; 14B sizes 2,048 rows 111 / 120; 3B
        sizes 4,096 rows 44 / 50) and not otherwise (7B 1,024 rows 32.7 / 30.5,
        1,536 rows 49.2 / 43.2; 3B 2,048 rows, 80 tiles for 74 pairs, 31.0 /
        27.5)."""
        if not (n >= FUSED_QKV_MIN_ROWS and x.dtype == torch.bfloat16 and self.qkv.weight.dtype == torch.bfloat16
                and self.qkv.bias is None and self.head_dim == ops.QKV_EPILOGUE_HEAD_DIM
                and 2 * cos.shape[1] == self.head_dim and x.stride(1) == 1 and x.stride(0) % 8 == 0
                and self.qkv.in_features % 8 == 0):
            return False
        pairs = max(1, ops.sm_count(x.device) // 2)
        tiles = ((n + 255) // 256) * ((self.qkv.out_features + 255) // 256)
        filled = tiles / (((tiles + pairs - 1) // pairs) * pairs)
        return filled >= 0.75 or (n >= 2 * FUSED_QKV_MIN_ROWS and filled >= 0.70)

    def attend(self, qkv, attn, ctx, step, g, k_layer, v_layer, page_stride) -> None:
        """bfloat16 with a head size the tensor-core kernels take: prompt
        portions go to the tcgen05 kernel (head size 128) or the mma.sync kernel
        (64), single tokens to the split decode kernel; anything else (float32,
        other head sizes) to the generic kernel."""
        common = (ctx.entry_q_start, ctx.entry_q_len, ctx.entry_ctx_start)
        if qkv.dtype != torch.bfloat16 or self.head_dim not in ops.FAST_ATTENTION_HEAD_DIMS:
            ops.attn_paged_generic(qkv, qkv.stride(0), attn, k_layer, v_layer, page_stride, ctx.page_size,
                                   ctx.block_tables[g], step.tile_entry, step.tile_q0, step.n_tiles, *common,
                                   self.n_heads, self.n_kv, self.head_dim, self.scale, self.window)
            return
        if step.n_chunk_tiles and self.head_dim == ops.UMMA_ATTENTION_HEAD_DIM:
            max_keys = min(ctx.max_ctx_len, self.window + 128) if self.window else ctx.max_ctx_len
            splits = ops.attn_prefill_umma_splits(step.n_umma_tiles, self.n_heads, max_keys)
            ops.attn_prefill_umma(qkv, qkv.stride(0), attn, k_layer, v_layer, page_stride, ctx.page_size,
                                  ctx.block_tables[g], step.umma_tile_entry, step.umma_tile_q0, step.n_umma_tiles,
                                  *common, self.n_heads, self.n_kv, self.head_dim, self.scale, self.window, splits,
                                  tile_rows=step.umma_tile_rows)
        elif step.n_chunk_tiles:
            ops.attn_prefill_bf16(qkv, qkv.stride(0), attn, k_layer, v_layer, page_stride, ctx.page_size,
                                  ctx.block_tables[g], step.chunk_tile_entry, step.chunk_tile_q0, step.n_chunk_tiles,
                                  *common, self.n_heads, self.n_kv, self.head_dim, self.scale, self.window)
        if step.n_decode:
            self.decode(qkv, attn, ctx, step, g, k_layer, v_layer, page_stride)

    def _share_by_tiles(self, step) -> bool:
        """Contexts of very different lengths (and no window that evens them
        out): the kernel that shares the tiles of all entries out evenly."""
        return (step.decode_skewed and step.n_decode <= ops.DECODE_EVEN_MAX_ENTRIES
                and not (self.window and self.window < 1024))

    def decode(self, qkv, attn, ctx, step, g, k_layer, v_layer, page_stride, prep=None) -> None:
        """The step's single tokens.  Contexts of about the same length: the keys
        of each are cut into as many parts as fill the GPU, and merged; with
        ``prep`` = (bias, cos, sin, slot map, partial sums or None) qkv is
        still the bare product and the kernel prepares q, k and v itself.
        Contexts of very different lengths: all their tiles are shared out
        evenly over the blocks."""
        max_keys = min(ctx.max_ctx_len, self.window) if self.window else ctx.max_ctx_len
        if prep is None and self._share_by_tiles(step):
            pieces = ops.attn_decode_pieces(self.n_heads, self.n_kv, self.head_dim, max_keys)
            rows = step.n_decode * self.n_heads * pieces
            part_o = torch.empty(rows * self.head_dim, dtype=torch.float32, device=qkv.device)
            part_ml = torch.empty(rows * 2, dtype=torch.float32, device=qkv.device)
            count = torch.empty(step.n_decode * self.n_heads, dtype=torch.int32, device=qkv.device)
            ops.attn_decode_even_bf16(qkv, attn, k_layer, v_layer, page_stride, ctx.page_size, ctx.block_tables[g],
                                      step.decode_entries, step.n_decode, ctx.entry_q_start, ctx.entry_q_len,
                                      ctx.entry_ctx_start, part_o, part_ml, count, self.n_heads, self.n_kv, self.head_dim,
                                      self.scale, self.window, pieces)
            return
        n_splits = ops.attn_decode_splits(step.n_decode, self.n_heads, self.n_kv, self.head_dim, max_keys)
        part_o = part_ml = None
        if n_splits > 1:
            rows = step.n_decode * self.n_heads * n_splits
            part_o = torch.empty(rows * self.head_dim, dtype=torch.float32, device=qkv.device)
            part_ml = torch.empty(rows * 2, dtype=torch.float32, device=qkv.device)
        meta = (k_layer, v_layer, page_stride, ctx.page_size, ctx.block_tables[g], step.decode_entries, step.n_decode,
                ctx.entry_q_start, ctx.entry_q_len, ctx.entry_ctx_start, part_o, part_ml,
                self.n_heads, self.n_kv, self.head_dim, self.scale, self.window, n_splits)
        if prep is None:
            ops.attn_decode_bf16(qkv, qkv.stride(0), attn, *meta)
        else:
            bias, cos, sin, slot_map, partials = prep
            ops.attn_decode_prep_bf16(qkv, bias, cos, sin, slot_map, partials, attn, *meta)


register_part("mixer", "gqa_attention", GQAttention)
