"""Python entry points of the hand-written CUDA kernels.

Each function takes torch tensors that already live on the GPU, checks what
the kernel cannot check itself, and launches on torch's current stream through
the C interface of the kernel library.  There is no other implementation
behind these functions: a tensor that is not on a CUDA device, or a library
that cannot be built, raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .build import library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong

#: kernels of this library launched since import (library matrix products are not counted)
launch_count = 0

_ERRORS = {100001: "unsupported size or element type", 100002: "misaligned pointer or stride"}


class KernelError(RuntimeError):
    pass


_sigs_done = False


def _lib():
    global _sigs_done
    lib = library()
    if not _sigs_done:
        lib.ifx_embed_gather.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.ifx_add_rmsnorm.argtypes = [c_void_p, c_void_p, c_int, c_int, c_ll, c_void_p, c_float, c_void_p,
                                        c_int, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.ifx_swiglu.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.ifx_convert.argtypes = [c_void_p, c_int, c_void_p, c_int, c_ll, c_void_p]
        lib.ifx_rope_table.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
        lib.ifx_qkv_rope_kv_write.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                              c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                              c_int, c_void_p]
        lib.ifx_gemm_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_void_p]
        lib.ifx_attn_paged_generic.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_int, c_void_p, c_void_p, c_ll, c_int,
                                               c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                               c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p]
        lib.ifx_attn_prefill_bf16.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int,
                                              c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                              c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p]
        lib.ifx_attn_decode_bf16.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int,
                                             c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
        lib.ifx_attn_decode_prep_bf16.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int,
                                                  c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                                  c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int,
                                                  c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
        lib.ifx_attn_decode_prep_bf16.restype = c_int
        lib.ifx_attn_decode_even_bf16.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int,
                                                  c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                                  c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int,
                                                  c_void_p, c_void_p]
        lib.ifx_attn_decode_even_bf16.restype = c_int
        lib.ifx_attn_decode_even_pieces.argtypes = [c_int, c_int, c_int, c_int]
        lib.ifx_attn_decode_even_pieces.restype = c_int
        lib.ifx_gemv_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_ll,
                                      c_int, c_int, c_void_p]
        lib.ifx_gemm_umma.argtypes = [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int,
                                      c_void_p, c_void_p]
        lib.ifx_gemm_umma.restype = c_int
        lib.ifx_gemm_umma_skinny.argtypes = [c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_ll, c_int, c_int, c_int, c_int,
                                             c_void_p, c_void_p]
        lib.ifx_gemm_umma_skinny.restype = c_int
        lib.ifx_gemm_umma_qkv.argtypes = [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
        lib.ifx_gemm_umma_qkv.restype = c_int
        lib.ifx_gemm_umma_skinny_parts.argtypes = [c_int, c_int]
        lib.ifx_gemm_umma_skinny_parts.restype = c_int
        lib.ifx_gemv_bf16_plan.argtypes = [c_int, c_int, c_int]
        lib.ifx_gemv_bf16_plan.restype = c_int
        lib.ifx_attn_decode_plan.argtypes = [c_int, c_int, c_int, c_int, c_int]
        lib.ifx_attn_decode_plan.restype = c_int
        lib.ifx_attn_prefill_umma.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int,
                                              c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                              c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p,
                                              c_void_p, c_int, c_int, c_int, c_void_p]
        lib.ifx_attn_prefill_umma_plan.argtypes = [c_int, c_int, c_int]
        lib.ifx_attn_prefill_umma_plan.restype = c_int
        lib.ifx_argmax.argtypes = [c_void_p, c_ll, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p]
        lib.ifx_apply_penalties.argtypes = [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                            c_void_p, c_int, c_int, c_void_p]
        lib.ifx_apply_penalties_ring.argtypes = [c_void_p, c_ll, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 c_void_p, c_void_p, c_int, c_int, c_void_p]
        lib.ifx_apply_penalties_ring.restype = c_int
        lib.ifx_ring_append.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
        lib.ifx_ring_append.restype = c_int
        lib.ifx_sample.argtypes = [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_int, c_int, c_void_p]
        for name in ("ifx_embed_gather", "ifx_add_rmsnorm", "ifx_swiglu", "ifx_convert", "ifx_rope_table",
                     "ifx_qkv_rope_kv_write", "ifx_gemm_f32", "ifx_attn_paged_generic", "ifx_argmax",
                     "ifx_attn_prefill_bf16", "ifx_attn_decode_bf16", "ifx_gemv_bf16", "ifx_attn_prefill_umma",
                     "ifx_apply_penalties", "ifx_sample"):
            getattr(lib, name).restype = c_int
        _sigs_done = True
    return lib


def _check(code: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if code != 0:
        msg = _ERRORS.get(code)
        if msg is None:
            msg = f"CUDA error {code}"
            try:
                torch.cuda.synchronize()
            except RuntimeError as e:   # surfaces the sticky error text
                msg += f" ({e})"
        raise KernelError(f"{what}: {msg}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernel operands must be CUDA tensors (there is no CPU path)")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported element type {t.dtype}") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


# ------------------------------------------------------------------ elementwise
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, :] = float32(table[ids[t], :]); ids int32 [N], out float32 [N, H]."""
    n, (vocab, hidden) = ids.numel(), table.shape
    _need(ids.dtype == torch.int32 and out.dtype == torch.float32, "embed_gather: ids int32, out float32")
    _need(table.is_contiguous() and out.is_contiguous() and tuple(out.shape) == (n, hidden),
          "embed_gather: contiguous table and out [N, H]")
    _check(_lib().ifx_embed_gather(_ptr(table), _code(table), _ptr(ids), _ptr(out), n, hidden, vocab, _stream()),
           "embed_gather")
    return out


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
                n_partials: int = 1) -> Optional[torch.Tensor]:
    """residual (float32 [N, H]) += delta; out = RMSNorm(residual) * weight.

    With ``rows`` (int32 [R]) only those rows are normed into out [R, H] and
    the residual is left untouched.  ``delta`` may be None; with
    ``n_partials`` > 1 it is [P, N, H] float32 partial sums.  ``out`` may be
    None (only the sum is stored)."""
    n, hidden = residual.shape
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "add_rmsnorm: residual float32 contiguous")
    _need(weight.dtype == torch.float32 and weight.numel() == hidden, "add_rmsnorm: weight float32 [H]")
    n_rows = rows.numel() if rows is not None else n
    if rows is not None:
        _need(rows.dtype == torch.int32, "add_rmsnorm: rows int32")
    pstride = 0
    if delta is not None:
        _need(delta.is_contiguous(), "add_rmsnorm: delta contiguous")
        if n_partials > 1:
            _need(tuple(delta.shape) == (n_partials, n, hidden), "add_rmsnorm: partials [P, N, H]")
            pstride = n * hidden
        else:
            _need(tuple(delta.shape) == (n, hidden), "add_rmsnorm: delta [N, H]")
    if out is not None:
        _need(out.is_contiguous() and tuple(out.shape) == (n_rows, hidden), "add_rmsnorm: out [rows, H]")
    dd = _code(delta) if delta is not None else F32
    od = _code(out) if out is not None else F32
    _check(_lib().ifx_add_rmsnorm(_ptr(residual), _ptr(delta), dd, n_partials, pstride, _ptr(weight), float(eps),
                                  _ptr(out), od, _ptr(rows), n_rows, hidden, 0 if rows is not None else 1,
                                  _stream()), "add_rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[m, i] = silu(gate_up[m, i]) * gate_up[m, I + i]."""
    m, two_i = gate_up.shape
    _need(two_i % 2 == 0 and tuple(out.shape) == (m, two_i // 2) and out.dtype == gate_up.dtype,
          "swiglu: gate_up [M, 2I], out [M, I] of the same type")
    _need(gate_up.is_contiguous() and out.is_contiguous(), "swiglu: contiguous operands")
    _check(_lib().ifx_swiglu(_ptr(gate_up), _ptr(out), _code(out), m, two_i // 2, _stream()), "swiglu")
    return out


def convert(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    _need(src.is_contiguous() and dst.is_contiguous() and src.numel() == dst.numel(), "convert: same size, contiguous")
    _check(_lib().ifx_convert(_ptr(src), _code(src), _ptr(dst), _code(dst), src.numel(), _stream()), "convert")
    return dst


# ----------------------------------------------------------------------- rotary
def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> None:
    """cos/sin [N, half] float32 of positions[t] * inv_freq[i] (inv_freq float64 [half])."""
    n, half = positions.numel(), inv_freq.numel()
    _need(positions.dtype == torch.int32 and inv_freq.dtype == torch.float64, "rope_table: int32 positions, float64 inv_freq")
    _need(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
          and tuple(cos.shape) == (n, half) and tuple(sin.shape) == (n, half), "rope_table: cos/sin float32 [N, half]")
    _check(_lib().ifx_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(cos), _ptr(sin), n, half, _stream()),
           "rope_table")


def qkv_rope_kv_write(qkv: torch.Tensor, bias: Optional[torch.Tensor], cos: torch.Tensor, sin: torch.Tensor,
                      slot_map: Optional[torch.Tensor], k_layer: Optional[torch.Tensor],
                      v_layer: Optional[torch.Tensor], page_stride: int, page_size: int,
                      n_heads: int, n_kv: int, head_dim: int, partials: Optional[torch.Tensor] = None) -> None:
    """Bias add, rotate-half rotation of q (in place) and k, and the write of k
    and v into the paged cache at ``slot_map`` (page * page_size + offset).
    With ``partials`` (float32 [S, N, width], bfloat16 qkv, full rotation, head
    size a multiple of 16) the rows are the sums of the S slices instead of
    qkv's content, and qkv only receives the rotated q."""
    n, width = qkv.shape
    _need(qkv.is_contiguous() and width == (n_heads + 2 * n_kv) * head_dim, "qkv_rope_kv_write: qkv [N, (nh + 2 nkv) hd]")
    rot_dim = 2 * cos.shape[1]
    _need(tuple(cos.shape) == tuple(sin.shape) and cos.shape[0] == n and cos.dtype == torch.float32
          and cos.is_contiguous() and sin.is_contiguous(), "qkv_rope_kv_write: cos/sin float32 [N, rot/2]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == width, "qkv_rope_kv_write: bias float32 [width]")
    if n_kv:
        _need(slot_map is not None and slot_map.dtype == torch.int32 and slot_map.numel() == n,
              "qkv_rope_kv_write: slot_map int32 [N]")
        _need(k_layer.dtype == qkv.dtype and v_layer.dtype == qkv.dtype, "qkv_rope_kv_write: cache of qkv's type")
    n_partials = 0
    if partials is not None:
        _need(partials.dtype == torch.float32 and partials.is_contiguous() and partials.dim() == 3
              and tuple(partials.shape[1:]) == (n, width) and qkv.dtype == torch.bfloat16
              and rot_dim == head_dim and head_dim % 16 == 0, "qkv_rope_kv_write: partial sums float32 [S, N, width]")
        n_partials = partials.shape[0]
    _check(_lib().ifx_qkv_rope_kv_write(_ptr(qkv), _code(qkv), _ptr(bias), _ptr(cos), _ptr(sin), rot_dim,
                                        _ptr(slot_map) if n_kv else None, _ptr(k_layer) if n_kv else None,
                                        _ptr(v_layer) if n_kv else None, page_stride, page_size, n, n_heads, n_kv,
                                        head_dim, _ptr(partials), n_partials, _stream()), "qkv_rope_kv_write")


# --------------------------------------------------------------- matrix product
def gemm_f32(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T + bias, all float32, plain FFMA."""
    m, k = a.shape
    n = w.shape[0]
    _need(a.dtype == torch.float32 and w.dtype == torch.float32 and out.dtype == torch.float32, "gemm_f32: float32")
    _need(w.shape[1] == k and w.is_contiguous() and tuple(out.shape) == (m, n), "gemm_f32: shapes")
    _need(a.stride(1) == 1 and out.stride(1) == 1, "gemm_f32: unit inner strides")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemm_f32: bias float32 [N]")
    _check(_lib().ifx_gemm_f32(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, a.stride(0) if m > 1 else k,
                               out.stride(0) if m > 1 else n, _stream()), "gemm_f32")
    return out


GEMV_MAX_ROWS = 16


def gemv_bf16(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
              swiglu: bool = False, k_splits: int = 1) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T (+ bias) for M <= 16, bfloat16 operands,
    float32 accumulation, bfloat16 or float32 result.  With ``swiglu`` w is
    [2N, K] = [gate; up] and out = silu(x gate^T) * (x up^T).  With
    ``k_splits`` > 1 out is float32 [k_splits, M, N]: slice s is the sum over the
    s-th part of K and the caller adds the slices.  ``w`` is a parameter: the
    kernel starts to read it before the kernel launched before it has finished,
    so it must not be that kernel's output."""
    m, k = x.shape
    n = out.shape[-1]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous(), "gemv_bf16: bfloat16 operands")
    _need(w.shape == ((2 * n if swiglu else n), k), "gemv_bf16: shapes")
    _need(m <= GEMV_MAX_ROWS and k % 8 == 0, f"gemv_bf16: at most {GEMV_MAX_ROWS} rows and K a multiple of 8")
    if k_splits > 1:
        _need(tuple(out.shape) == (k_splits, m, n) and out.is_contiguous() and out.dtype == torch.float32
              and not swiglu, "gemv_bf16: partial sums are float32 [k_splits, M, N]")
        ldo = n
    else:
        _need(out.dim() == 2 and out.shape[0] == m and out.stride(1) == 1, "gemv_bf16: out [M, N]")
        ldo = out.stride(0) if m > 1 else n
    _need(x.stride(1) == 1, "gemv_bf16: unit inner strides")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n and not swiglu, "gemv_bf16: bias float32 [N]")
    _check(_lib().ifx_gemv_bf16(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _code(out), m, n, k,
                                x.stride(0) if m > 1 else k, ldo, 1 if swiglu else 0, int(k_splits),
                                _stream()), "gemv_bf16")
    return out


def gemm_umma(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
              swiglu: bool = False) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T (+ bias) for many rows, on the tcgen05 tensor
    cores (TMA operands, accumulators in tensor memory), bfloat16 operands, float32
    accumulation, bfloat16 or float32 result.  With ``swiglu`` w is [2N, K] =
    [gate; up] and out = silu(x gate^T) * (x up^T), the activation applied in the
    product's epilogue.  Two SMs share each tile (cta_group::2).  A bounded wait
    that runs out sets the device's error flag (see :func:`check_device_errors`)."""
    m, k = x.shape
    n = out.shape[-1]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous(), "gemm_umma: bfloat16 operands")
    _need(w.shape == ((2 * n if swiglu else n), k), "gemm_umma: shapes")
    _need(out.dim() == 2 and out.shape[0] == m and out.stride(1) == 1 and x.stride(1) == 1,
          "gemm_umma: out [M, N], unit inner strides")
    _need(k % 8 == 0 and (m == 1 or x.stride(0) % 8 == 0), "gemm_umma: K and the row stride of x must be multiples of 8")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n and not swiglu, "gemm_umma: bias float32 [N]")
    _check(_lib().ifx_gemm_umma(_ptr(x), x.stride(0) if m > 1 else k, _ptr(w), _ptr(bias), _ptr(out), out.stride(0),
                                _code(out), m, n, k, 1 if swiglu else 0, _ptr(error_flag(x.device)), _stream()),
           "gemm_umma")
    return out


QKV_EPILOGUE_HEAD_DIM = 128     # the head size gemm_umma_qkv is written for


def gemm_umma_qkv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                  cos: torch.Tensor, sin: torch.Tensor, slot_map: Optional[torch.Tensor],
                  k_layer: Optional[torch.Tensor], v_layer: Optional[torch.Tensor], page_stride: int, page_size: int,
                  n_heads: int, n_kv: int) -> torch.Tensor:
    """The stacked q, k, v projection x[M, K] @ w[(nh + 2 nkv) * 128, K]^T of many
    rows on the tcgen05 tensor cores, with what stands between it and attention
    in its epilogue: bias, rotate-half rotation of the query and key heads
    (``cos``, ``sin`` float32 [M, 64]), the queries as bfloat16 into the first
    nh * 128 columns of ``q_out``'s rows, keys and values into the paged cache
    at ``slot_map`` (page * page_size + offset).  Head size 128 only."""
    m, k = x.shape
    hd = QKV_EPILOGUE_HEAD_DIM
    width = (n_heads + 2 * n_kv) * hd
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and tuple(w.shape) == (width, k),
          "gemm_umma_qkv: bfloat16 x [M, K], w [(nh + 2 nkv) * 128, K]")
    _need(q_out.dtype == torch.bfloat16 and q_out.dim() == 2 and q_out.shape[0] == m and q_out.shape[1] >= n_heads * hd
          and q_out.stride(1) == 1 and q_out.stride(0) % 8 == 0, "gemm_umma_qkv: q_out bfloat16 [M, >= nh * 128]")
    _need(k % 8 == 0 and x.stride(1) == 1 and (m == 1 or x.stride(0) % 8 == 0),
          "gemm_umma_qkv: K and the row stride of x must be multiples of 8")
    _need(tuple(cos.shape) == (m, hd // 2) and tuple(sin.shape) == (m, hd // 2) and cos.dtype == torch.float32
          and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous(),
          "gemm_umma_qkv: cos/sin float32 [M, 64]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == width, "gemm_umma_qkv: bias float32 [width]")
    if n_kv:
        _need(slot_map is not None and slot_map.dtype == torch.int32 and slot_map.numel() == m
              and k_layer.dtype == torch.bfloat16 and v_layer.dtype == torch.bfloat16,
              "gemm_umma_qkv: slot_map int32 [M], bfloat16 cache")
    _check(_lib().ifx_gemm_umma_qkv(_ptr(x), x.stride(0) if m > 1 else k, _ptr(w), _ptr(bias), _ptr(q_out), q_out.stride(0),
                                    _ptr(cos), _ptr(sin), _ptr(slot_map) if n_kv else None,
                                    _ptr(k_layer) if n_kv else None, _ptr(v_layer) if n_kv else None, page_stride,
                                    page_size, m, k, n_heads, n_kv, _ptr(error_flag(x.device)), _stream()), "gemm_umma_qkv")
    return q_out


SKINNY_MAX_ROWS = 256       # rows of x that gemm_umma_skinny takes


def gemm_umma_skinny_parts(n: int, k: int) -> int:
    """Into how many parts :func:`gemm_umma_skinny` cuts K for an [n, k] matrix."""
    key = ("skinny", n, k)
    if key not in _gemv_plans:
        s = int(_lib().ifx_gemm_umma_skinny_parts(n, k))
        if s < 1:
            raise KernelError(f"gemm_umma_skinny_parts: CUDA error {-s}")
        _gemv_plans[key] = s
    return _gemv_plans[key]


def gemm_umma_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Partial sums of x[M, K] @ w[N, K]^T for a few rows (up to
    SKINNY_MAX_ROWS), where the time goes to reading w once: out float32
    [S, M, N], S = ``gemm_umma_skinny_parts(N, K)`` parts of K, to be added by
    the consumer.  tcgen05 with the operands' places changed: 256 rows of w are
    the rows of a tile and the rows of x its columns."""
    m, k = x.shape
    s, m2, n = out.shape
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and tuple(w.shape) == (n, k),
          "gemm_umma_skinny: bfloat16 x [M, K], w [N, K]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and m2 == m and 1 <= m <= SKINNY_MAX_ROWS
          and s == gemm_umma_skinny_parts(n, k), "gemm_umma_skinny: out float32 [parts, M, N]")
    _need(k % 8 == 0 and x.stride(1) == 1 and (m == 1 or x.stride(0) % 8 == 0),
          "gemm_umma_skinny: K and the row stride of x must be multiples of 8")
    _check(_lib().ifx_gemm_umma_skinny(_ptr(x), x.stride(0) if m > 1 else k, _ptr(w), _ptr(out), n, m * n, m, n, k, s,
                                       _ptr(error_flag(x.device)), _stream()), "gemm_umma_skinny")
    return out


_gemv_plans = {}


def gemv_k_splits(n: int, k: int, max_splits: int = 8) -> int:
    """Into how many parts of K the weight-streaming kernel is best told to cut
    an [n, k] matrix when float32 partial sums are welcome: the kernel's own
    count of what keeps the GPU fullest.  It depends on the matrix only."""
    key = (n, k, max_splits)
    if key not in _gemv_plans:
        s = int(_lib().ifx_gemv_bf16_plan(n, k, max_splits))
        if s < 1:
            raise KernelError(f"gemv_k_splits: CUDA error {-s}")
        _gemv_plans[key] = s
    return _gemv_plans[key]


_sm_counts = {}


def sm_count(device) -> int:
    """SMs of the device (where a kernel's plan is made on the host)."""
    key = torch.device(device).index or 0
    if key not in _sm_counts:
        _sm_counts[key] = int(torch.cuda.get_device_properties(key).multi_processor_count)
    return _sm_counts[key]


_error_flags = {}


def error_flag(device) -> torch.Tensor:
    """The device word that kernels with bounded waits set when a wait runs out."""
    key = torch.device(device).index or 0
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


def check_device_errors(device) -> None:
    """Raise if a kernel reported that one of its bounded waits ran out (this
    reads one word back from the device, so it synchronises)."""
    key = torch.device(device).index or 0
    flag = _error_flags.get(key)
    if flag is not None:
        code = int(flag.item())
        if code != 0:
            flag.zero_()
            if code == 2:
                raise KernelError("decode attention met a context longer than the bound its scratch was sized for; "
                                  "its output is invalid")
            raise KernelError("a kernel gave up waiting on a barrier (bounded wait ran out); its output is invalid")


def matmul_library(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x[M, K] @ w[N, K]^T through the vendor library (cuBLAS via torch), bfloat16
    operands, float32 accumulation, bfloat16 or float32 result.  Stands where
    the reference calls cuBLAS (runtime/backends/cuda/native/cublas_gemm.cpp:84-102)."""
    _need(x.is_cuda and w.is_cuda, "matmul_library: CUDA tensors (there is no CPU path)")
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "matmul_library: bfloat16 operands")
    if out_dtype == torch.float32:
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    return torch.mm(x, w.t())


# -------------------------------------------------------------------- attention
def attn_paged_generic(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_layer: torch.Tensor,
                       v_layer: torch.Tensor, page_stride: int, page_size: int, block_tables: torch.Tensor,
                       tile_entry: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int,
                       entry_q_start: torch.Tensor, entry_q_len: torch.Tensor, entry_ctx_start: torch.Tensor,
                       n_heads: int, n_kv: int, head_dim: int, scale: float, window: int) -> torch.Tensor:
    """Causal grouped-query attention of new tokens over the paged cache.

    q: first element of the query rows (row stride ``q_stride`` elements, heads
    contiguous); out [N, n_heads * head_dim]; query tiles of 16 tokens are
    listed by tile_entry / tile_q0."""
    _need(block_tables.dtype == torch.int32 and block_tables.dim() == 2 and block_tables.stride(1) == 1,
          "attn: block_tables int32 [R, B]")
    for t in (tile_entry, tile_q0, entry_q_start, entry_q_len, entry_ctx_start):
        _need(t.dtype == torch.int32, "attn: int32 metadata")
    _need(out.is_contiguous() and out.dtype == q.dtype and k_layer.dtype == q.dtype, "attn: types")
    _need(1 <= head_dim <= 256, f"attention: head_dim {head_dim} is outside 1..256")
    _need(n_heads % n_kv == 0, "attention: n_heads must be a multiple of n_kv")
    _check(_lib().ifx_attn_paged_generic(_ptr(q), q_stride, _ptr(out), out.stride(0), _code(q), _ptr(k_layer),
                                         _ptr(v_layer), page_stride, page_size, _ptr(block_tables),
                                         block_tables.stride(0), _ptr(tile_entry), _ptr(tile_q0), n_tiles,
                                         _ptr(entry_q_start), _ptr(entry_q_len), _ptr(entry_ctx_start),
                                         n_heads, n_kv, head_dim, float(scale), int(window), _stream()),
           "attn_paged_generic")
    return out


FAST_ATTENTION_HEAD_DIMS = (64, 128)


def attn_prefill_bf16(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_layer: torch.Tensor,
                      v_layer: torch.Tensor, page_stride: int, page_size: int, block_tables: torch.Tensor,
                      tile_entry: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int,
                      entry_q_start: torch.Tensor, entry_q_len: torch.Tensor, entry_ctx_start: torch.Tensor,
                      n_heads: int, n_kv: int, head_dim: int, scale: float, window: int) -> torch.Tensor:
    """Tensor-core attention of prompt portions over the paged cache (bfloat16,
    head_dim 64 or 128); query tiles of 64 tokens listed by tile_entry / tile_q0."""
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_layer.dtype == torch.bfloat16,
          "attn_prefill_bf16: bfloat16 operands")
    _need(head_dim in FAST_ATTENTION_HEAD_DIMS, f"attn_prefill_bf16: head_dim {head_dim} not in {FAST_ATTENTION_HEAD_DIMS}")
    _need(block_tables.dtype == torch.int32 and block_tables.stride(1) == 1, "attn: block_tables int32 [R, B]")
    _check(_lib().ifx_attn_prefill_bf16(_ptr(q), q_stride, _ptr(out), out.stride(0), _ptr(k_layer), _ptr(v_layer),
                                        page_stride, page_size, _ptr(block_tables), block_tables.stride(0),
                                        _ptr(tile_entry), _ptr(tile_q0), n_tiles, _ptr(entry_q_start),
                                        _ptr(entry_q_len), _ptr(entry_ctx_start), n_heads, n_kv, head_dim,
                                        float(scale), int(window), _stream()), "attn_prefill_bf16")
    return out


UMMA_ATTENTION_HEAD_DIM = 128
UMMA_ATTENTION_TILE = 256          # tokens per query tile of attn_prefill_umma


def attn_prefill_umma(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_layer: torch.Tensor,
                      v_layer: torch.Tensor, page_stride: int, page_size: int, block_tables: torch.Tensor,
                      tile_entry: torch.Tensor, tile_q0: torch.Tensor, n_tiles: int,
                      entry_q_start: torch.Tensor, entry_q_len: torch.Tensor, entry_ctx_start: torch.Tensor,
                      n_heads: int, n_kv: int, head_dim: int, scale: float, window: int,
                      n_splits: int = 1, tile_rows: int = 256) -> torch.Tensor:
    """Attention of prompt portions with tcgen05.mma and tensor-memory
    accumulators (bfloat16, head_dim 128); query tiles of ``tile_rows`` = 256 or
    128 tokens listed by tile_entry / tile_q0 (a block takes a tile and a head;
    with 128 the tile's key tiles are dealt out to both halves of the block:
    twice the blocks, for steps whose tiles of 256 would leave SMs idle).  With ``n_splits`` > 1 the keys of every tile are cut
    into that many parts (see :func:`attn_prefill_umma_splits`), merged by a
    second kernel.  A bounded wait that runs out sets the device error flag
    (see :func:`check_device_errors`)."""
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_layer.dtype == torch.bfloat16,
          "attn_prefill_umma: bfloat16 operands")
    _need(head_dim == UMMA_ATTENTION_HEAD_DIM, f"attn_prefill_umma: head_dim {head_dim} is not 128")
    _need(block_tables.dtype == torch.int32 and block_tables.stride(1) == 1, "attn: block_tables int32 [R, B]")
    # The kernel reads the cache through a TMA tensor map, which wants to know how many pages lie behind page 0:
    # as many as fit between the view's start and the end of the storage it is a view of.
    n_elems = k_layer.untyped_storage().nbytes() // k_layer.element_size()
    last = max(k_layer.storage_offset(), v_layer.storage_offset()) + n_kv * page_size * head_dim
    num_pages = (n_elems - last) // page_stride + 1 if n_elems >= last else 0
    _need(num_pages >= 1, "attn_prefill_umma: k_layer / v_layer are not views of page 0 of a paged pool")
    part_o = part_ml = None
    global launch_count
    if n_splits > 1:
        rows = n_tiles * n_heads * n_splits * UMMA_ATTENTION_TILE
        part_o = torch.empty(rows * head_dim, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(rows * 2, dtype=torch.float32, device=q.device)
        launch_count += 1          # the merge kernel
    _check(_lib().ifx_attn_prefill_umma(_ptr(q), q_stride, _ptr(out), out.stride(0), _ptr(k_layer), _ptr(v_layer),
                                        page_stride, page_size, _ptr(block_tables), block_tables.stride(0),
                                        _ptr(tile_entry), _ptr(tile_q0), n_tiles, _ptr(entry_q_start),
                                        _ptr(entry_q_len), _ptr(entry_ctx_start), n_heads, n_kv, head_dim,
                                        float(scale), int(window), _ptr(error_flag(q.device)), _ptr(part_o),
                                        _ptr(part_ml), int(n_splits), int(num_pages), int(tile_rows), _stream()),
           "attn_prefill_umma")
    return out


def attn_prefill_umma_splits(n_tiles: int, n_heads: int, max_keys: int) -> int:
    """Into how many parts :func:`attn_prefill_umma` is best told to cut the keys
    of its query tiles (the kernel's own count: 1 when the tiles fill the GPU)."""
    return max(1, int(_lib().ifx_attn_prefill_umma_plan(n_tiles, n_heads, (max_keys + 63) // 64)))


def attn_decode_bf16(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_layer: torch.Tensor,
                     v_layer: torch.Tensor, page_stride: int, page_size: int, block_tables: torch.Tensor,
                     dec_entries: torch.Tensor, n_dec: int, entry_q_start: torch.Tensor,
                     entry_q_len: torch.Tensor, entry_ctx_start: torch.Tensor, part_o: Optional[torch.Tensor],
                     part_ml: Optional[torch.Tensor], n_heads: int, n_kv: int, head_dim: int, scale: float,
                     window: int, n_splits: int) -> torch.Tensor:
    """Tensor-core attention of single decoded tokens (entries listed in
    dec_entries), the keys split ``n_splits`` ways and merged.  Scratch:
    part_o float32 [n_dec * n_heads * n_splits * head_dim], part_ml float32
    [n_dec * n_heads * n_splits * 2]."""
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_layer.dtype == torch.bfloat16,
          "attn_decode_bf16: bfloat16 operands")
    _need(head_dim in FAST_ATTENTION_HEAD_DIMS, f"attn_decode_bf16: head_dim {head_dim} not in {FAST_ATTENTION_HEAD_DIMS}")
    _need(block_tables.dtype == torch.int32 and block_tables.stride(1) == 1, "attn: block_tables int32 [R, B]")
    if n_splits > 1:
        _need(part_o is not None and part_o.dtype == torch.float32
              and part_o.numel() >= n_dec * n_heads * n_splits * head_dim
              and part_ml is not None and part_ml.dtype == torch.float32
              and part_ml.numel() >= n_dec * n_heads * n_splits * 2, "attn_decode_bf16: scratch too small")
    global launch_count
    if n_splits > 1:
        launch_count += 1          # the merge kernel
    _check(_lib().ifx_attn_decode_bf16(_ptr(q), q_stride, _ptr(out), out.stride(0), _ptr(k_layer), _ptr(v_layer),
                                       page_stride, page_size, _ptr(block_tables), block_tables.stride(0),
                                       _ptr(dec_entries), n_dec, _ptr(entry_q_start), _ptr(entry_q_len),
                                       _ptr(entry_ctx_start), _ptr(part_o), _ptr(part_ml), n_heads, n_kv, head_dim,
                                       float(scale), int(window), int(n_splits), _stream()), "attn_decode_bf16")
    return out


def attn_decode_prep_bf16(qkv: torch.Tensor, bias: Optional[torch.Tensor], cos: torch.Tensor, sin: torch.Tensor,
                          slot_map: Optional[torch.Tensor], partials: Optional[torch.Tensor], out: torch.Tensor,
                          k_layer: torch.Tensor, v_layer: torch.Tensor, page_stride: int, page_size: int,
                          block_tables: torch.Tensor, dec_entries: torch.Tensor, n_dec: int,
                          entry_q_start: torch.Tensor, entry_q_len: torch.Tensor, entry_ctx_start: torch.Tensor,
                          part_o: Optional[torch.Tensor], part_ml: Optional[torch.Tensor], n_heads: int, n_kv: int,
                          head_dim: int, scale: float, window: int, n_splits: int) -> torch.Tensor:
    """:func:`attn_decode_bf16` for a step of single tokens only, with the work
    of :func:`qkv_rope_kv_write` folded into the attention kernel: ``qkv`` is
    the product's output before bias and rotation (or ``partials``, float32
    [S, N, width], holds it as partial sums and qkv's content is not read);
    the kernel rotates its own query heads and writes the token's key and
    value into the cache (``slot_map`` None: the layer writes none) before it
    reads them.  Every row of qkv must be one of the decoded entries."""
    n, width = qkv.shape
    _need(qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_layer.dtype == torch.bfloat16
          and qkv.is_contiguous() and width == (n_heads + 2 * n_kv) * head_dim and n == n_dec,
          "attn_decode_prep_bf16: qkv bfloat16 [n_dec, (nh + 2 nkv) hd]")
    _need(head_dim in FAST_ATTENTION_HEAD_DIMS, f"attn_decode_prep_bf16: head_dim {head_dim} not in {FAST_ATTENTION_HEAD_DIMS}")
    _need(tuple(cos.shape) == (n, head_dim // 2) and tuple(sin.shape) == (n, head_dim // 2) and cos.dtype == torch.float32
          and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous(),
          "attn_decode_prep_bf16: cos/sin float32 [N, head_dim / 2]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == width), "attn_decode_prep_bf16: bias float32 [width]")
    _need(slot_map is None or (slot_map.dtype == torch.int32 and slot_map.numel() == n), "attn_decode_prep_bf16: slot_map int32 [N]")
    _need(block_tables.dtype == torch.int32 and block_tables.stride(1) == 1, "attn: block_tables int32 [R, B]")
    n_partials = 0
    if partials is not None:
        _need(partials.dtype == torch.float32 and partials.is_contiguous() and partials.dim() == 3
              and tuple(partials.shape[1:]) == (n, width), "attn_decode_prep_bf16: partial sums float32 [S, N, width]")
        n_partials = partials.shape[0]
    if n_splits > 1:
        _need(part_o is not None and part_o.dtype == torch.float32
              and part_o.numel() >= n_dec * n_heads * n_splits * head_dim
              and part_ml is not None and part_ml.dtype == torch.float32
              and part_ml.numel() >= n_dec * n_heads * n_splits * 2, "attn_decode_prep_bf16: scratch too small")
    global launch_count
    if n_splits > 1:
        launch_count += 1          # the merge kernel
    _check(_lib().ifx_attn_decode_prep_bf16(_ptr(qkv), qkv.stride(0), _ptr(out), out.stride(0), _ptr(k_layer),
                                            _ptr(v_layer), page_stride, page_size, _ptr(block_tables),
                                            block_tables.stride(0), _ptr(dec_entries), n_dec, _ptr(entry_q_start),
                                            _ptr(entry_q_len), _ptr(entry_ctx_start), _ptr(part_o), _ptr(part_ml),
                                            n_heads, n_kv, head_dim, float(scale), int(window), int(n_splits),
                                            _ptr(bias), _ptr(cos), _ptr(sin), _ptr(slot_map), _ptr(partials),
                                            n_partials, n, _stream()), "attn_decode_prep_bf16")
    return out


_decode_plans = {}


def attn_decode_splits(n_dec: int, n_heads: int, n_kv: int, head_dim: int, max_keys: int) -> int:
    """Into how many parts :func:`attn_decode_bf16` is best told to cut the keys
    (the kernel's own count: every block has a place on the GPU at once)."""
    key = (n_dec, n_heads, n_kv, head_dim, (max_keys + 63) // 64)
    if key not in _decode_plans:
        if len(_decode_plans) > 65536:
            _decode_plans.clear()
        s = int(_lib().ifx_attn_decode_plan(n_dec, n_heads, n_kv, head_dim, max_keys))
        if s < 1:
            raise KernelError(f"attn_decode_splits: CUDA error {-s}")
        _decode_plans[key] = s
    return _decode_plans[key]


DECODE_EVEN_MAX_ENTRIES = 1024        # single tokens per call of attn_decode_even_bf16


def attn_decode_pieces(n_heads: int, n_kv: int, head_dim: int, max_keys: int) -> int:
    """Pieces per (entry, head) that :func:`attn_decode_even_bf16`'s scratch must
    have room for when no entry sees more than ``max_keys`` keys."""
    key = ("even", n_heads, n_kv, head_dim, (max_keys + 63) // 64)
    if key not in _decode_plans:
        if len(_decode_plans) > 65536:
            _decode_plans.clear()
        s = int(_lib().ifx_attn_decode_even_pieces(n_heads, n_kv, head_dim, max_keys))
        if s < 1:
            raise KernelError(f"attn_decode_pieces: CUDA error {-s}")
        _decode_plans[key] = s
    return _decode_plans[key]


def attn_decode_even_bf16(q: torch.Tensor, out: torch.Tensor, k_layer: torch.Tensor, v_layer: torch.Tensor,
                          page_stride: int, page_size: int, block_tables: torch.Tensor, dec_entries: torch.Tensor,
                          n_dec: int, entry_q_start: torch.Tensor, entry_q_len: torch.Tensor,
                          entry_ctx_start: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor,
                          piece_count: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, scale: float, window: int,
                          max_pieces: int) -> torch.Tensor:
    """Tensor-core attention of single decoded tokens (entries listed in
    dec_entries, at most DECODE_EVEN_MAX_ENTRIES) for steps whose contexts
    differ much in length: the 64-key tiles of all entries are shared out
    evenly over the blocks the GPU holds, so the longest context does not set
    the time; what several blocks share is merged by a second kernel.
    ``max_pieces`` from :func:`attn_decode_pieces`; scratch part_o float32
    [n_dec * n_heads * max_pieces * head_dim], part_ml float32 [... * 2],
    piece_count int32 [n_dec * n_heads].  A context beyond the bound that
    max_pieces was made for sets the device error flag."""
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_layer.dtype == torch.bfloat16,
          "attn_decode_even_bf16: bfloat16 operands")
    _need(head_dim in FAST_ATTENTION_HEAD_DIMS, f"attn_decode_even_bf16: head_dim {head_dim} not in {FAST_ATTENTION_HEAD_DIMS}")
    _need(block_tables.dtype == torch.int32 and block_tables.stride(1) == 1, "attn: block_tables int32 [R, B]")
    _need(1 <= n_dec <= DECODE_EVEN_MAX_ENTRIES, f"attn_decode_even_bf16: 1 to {DECODE_EVEN_MAX_ENTRIES} entries")
    _need(part_o.dtype == torch.float32 and part_o.numel() >= n_dec * n_heads * max_pieces * head_dim
          and part_ml.dtype == torch.float32 and part_ml.numel() >= n_dec * n_heads * max_pieces * 2
          and piece_count.dtype == torch.int32 and piece_count.numel() >= n_dec * n_heads,
          "attn_decode_even_bf16: scratch too small")
    global launch_count
    launch_count += 1          # the merge kernel
    _check(_lib().ifx_attn_decode_even_bf16(_ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_layer), _ptr(v_layer),
                                            page_stride, page_size, _ptr(block_tables), block_tables.stride(0),
                                            _ptr(dec_entries), n_dec, _ptr(entry_q_start), _ptr(entry_q_len),
                                            _ptr(entry_ctx_start), _ptr(part_o), _ptr(part_ml), _ptr(piece_count), n_heads,
                                            n_kv, head_dim, float(scale), int(window), int(max_pieces),
                                            _ptr(error_flag(q.device)), _stream()), "attn_decode_even_bf16")
    return out


# --------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] = lowest index of the maximum of logits[r, :] (float32 [R, V])."""
    r, v = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32 and out.numel() >= r,
          "argmax: float32 logits, int32 out")
    # a wide row is cut into slices with a block each (then a second launch picks among them)
    parts = min(64, v // 2048) if r <= 65535 else 1
    part = None
    global launch_count
    if parts > 1:
        part = torch.empty((r, parts, 2), dtype=torch.int32, device=logits.device)
        launch_count += 1
    _check(_lib().ifx_argmax(_ptr(logits), logits.stride(0), _ptr(out), r, v, _ptr(part), parts, _stream()), "argmax")
    return out


def apply_penalties(logits: torch.Tensor, recent_ids: torch.Tensor, recent_counts: torch.Tensor,
                    n_recent: torch.Tensor, rep: torch.Tensor, freq: torch.Tensor, pres: torch.Tensor) -> None:
    r, v = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "penalties: float32 logits")
    _need(recent_ids.dtype == torch.int32 and recent_counts.dtype == torch.int32 and n_recent.dtype == torch.int32
          and recent_ids.is_contiguous() and recent_counts.is_contiguous() and recent_ids.shape[0] == r
          and recent_ids.shape == recent_counts.shape, "penalties: int32 [R, W] ids and counts")
    for t in (rep, freq, pres):
        _need(t.dtype == torch.float32 and t.numel() == r, "penalties: float32 [R] parameters")
    _check(_lib().ifx_apply_penalties(_ptr(logits), logits.stride(0), _ptr(recent_ids), _ptr(recent_counts),
                                      _ptr(n_recent), recent_ids.shape[1], _ptr(rep), _ptr(freq), _ptr(pres), r, v,
                                      _stream()), "apply_penalties")


def apply_penalties_ring(logits: torch.Tensor, ring: torch.Tensor, totals: torch.Tensor, slots: torch.Tensor,
                         last_n: torch.Tensor, rep: torch.Tensor, freq: torch.Tensor, pres: torch.Tensor) -> None:
    """The penalties of :func:`apply_penalties` over each row's latest tokens,
    read from rings on the device: ``ring`` int32 [n_slots, ring_size] holds a
    request's tokens in order of arrival, written round and round,
    ``totals[slot]`` how many were written in all; row r is the request in
    ``slots[r]`` (negative: leave the row alone) and counts its latest
    ``last_n[r]`` tokens (at most ring_size)."""
    r, v = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "apply_penalties_ring: float32 logits")
    _need(ring.dtype == torch.int32 and ring.dim() == 2 and ring.is_contiguous() and totals.dtype == torch.int32
          and totals.numel() >= ring.shape[0], "apply_penalties_ring: ring int32 [slots, size], totals int32 [slots]")
    _need(slots.dtype == torch.int32 and slots.numel() >= r and last_n.dtype == torch.int32 and last_n.numel() >= r
          and all(t.dtype == torch.float32 and t.numel() >= r for t in (rep, freq, pres)),
          "apply_penalties_ring: one slot, window and penalty triple per row")
    _check(_lib().ifx_apply_penalties_ring(_ptr(logits), logits.stride(0), _ptr(ring), ring.shape[1], _ptr(totals),
                                           _ptr(slots), _ptr(last_n), _ptr(rep), _ptr(freq), _ptr(pres), r, v, _stream()),
           "apply_penalties_ring")


def ring_append(ring: torch.Tensor, totals: torch.Tensor, slots: torch.Tensor, ids: torch.Tensor) -> None:
    """ids[r] becomes the next token of the request in slots[r] (negative: skipped)."""
    _need(ring.dtype == torch.int32 and ring.dim() == 2 and ring.is_contiguous() and totals.dtype == torch.int32
          and slots.dtype == torch.int32 and ids.dtype == torch.int32 and slots.numel() >= ids.numel(),
          "ring_append: int32 operands")
    _check(_lib().ifx_ring_append(_ptr(ring), ring.shape[1], _ptr(totals), _ptr(slots), _ptr(ids), ids.numel(), _stream()),
           "ring_append")


def sample(logits: torch.Tensor, weights: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, min_p: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor,
           out: torch.Tensor) -> torch.Tensor:
    """One token per row: argmax where temperature <= 0, else a draw from
    softmax(logits / T) restricted by top-k / top-p / min-p.  ``weights`` is
    float32 scratch of logits' shape; seeds / counters are int64 (read as
    unsigned)."""
    r, v = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "sample: float32 logits")
    _need(weights.dtype == torch.float32 and weights.is_contiguous() and weights.numel() >= r * v, "sample: scratch")
    _need(temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and min_p.dtype == torch.float32
          and top_k.dtype == torch.int32 and seeds.dtype == torch.int64 and counters.dtype == torch.int64
          and out.dtype == torch.int32, "sample: parameter types")
    _check(_lib().ifx_sample(_ptr(logits), logits.stride(0), _ptr(weights), _ptr(temperature), _ptr(top_k),
                             _ptr(top_p), _ptr(min_p), _ptr(seeds), _ptr(counters), _ptr(out), r, v, _stream()),
           "sample")
    return out
