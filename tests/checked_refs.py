"""The two references of the kernels, held against each other.

Every function here has the signature of its namesake in ``kernel_refs.py``
(plain PyTorch) and returns what that one returns, after running the host-side
C++ reference (``inferflux_b200/csrc/host_reference``, through
``inferflux_b200.kernels.host_reference``) on float32 copies of the same inputs
and checking that the two agree.  A kernel test that compares with these
functions therefore compares three implementations written separately: the CUDA
kernel, the PyTorch restatement and the C++ loops.
"""
from __future__ import annotations

import torch

import kernel_refs as _py
from inferflux_b200.kernels import host_reference as _cc

uniform01 = _py.uniform01
rope_table = _py.rope_table
convert = _py.convert
gemm_f32 = _py.gemm_f32
embed_gather = _py.embed_gather
argmax = _py.argmax


def _agree(a, b, what, stored_dtype=torch.float32):
    """a: the PyTorch reference's result (maybe rounded to ``stored_dtype``), b: the C++ one in float32."""
    a, b = a.double().cpu(), b.double().cpu()
    tol = 2e-5 if stored_dtype == torch.float32 else 2.0 ** -8 * 1.1
    err = float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))
    assert err <= tol, f"the PyTorch and the C++ reference of {what} differ by {err:.3e}"


def _f(t):
    return None if t is None else t.detach().to("cpu", torch.float32).contiguous().clone()


def _i(t):
    return None if t is None else t.detach().to("cpu", torch.int32).contiguous()


def add_rmsnorm(residual, delta, weight, eps, out, rows=None, n_partials=1):
    res_c, out_c = _f(residual), (None if out is None else torch.empty(out.shape, dtype=torch.float32))
    _cc.add_rmsnorm(res_c, _f(delta), _f(weight), eps, out_c, _i(rows), n_partials)
    _py.add_rmsnorm(residual, delta, weight, eps, out, rows, n_partials)
    _agree(residual, res_c, "add + norm (residual)")
    if out is not None:
        _agree(out, out_c, "add + norm (normed rows)", out.dtype)
    return out


def swiglu(gate_up, out):
    out_c = torch.empty(out.shape, dtype=torch.float32)
    _cc.swiglu(_f(gate_up), out_c)
    _py.swiglu(gate_up, out)
    _agree(out, out_c, "SwiGLU", out.dtype)
    return out


def gemv_bf16(x, w, bias, out, swiglu=False, k_splits=1):
    _py.gemv_bf16(x, w, bias, out, swiglu, k_splits)
    if x.shape[0] * w.shape[0] * x.shape[1] <= 2e8:              # the C++ loops take a minute on the largest case
        n = w.shape[0]
        y = torch.empty((x.shape[0], n), dtype=torch.float32)
        _cc.gemm(_f(x), _f(w), None if swiglu else _f(bias), y)
        if swiglu:
            act = torch.empty((x.shape[0], n // 2), dtype=torch.float32)
            _cc.swiglu(y, act)
            y = act
        _agree(out.float().sum(0) if k_splits > 1 else out, y, "the product for a few rows", out.dtype)
    return out


def qkv_rope_kv_write(qkv, bias, cos, sin, slot_map, k_layer, v_layer, page_stride, page_size, n_heads, n_kv, head_dim):
    # the cache of the C++ side: a float32 copy of the whole pool that k_layer / v_layer are views of
    pool = k_layer._base if k_layer._base is not None else k_layer
    pool_c = _f(pool)
    k_off, v_off = k_layer.storage_offset(), v_layer.storage_offset()
    k_c = torch.as_strided(pool_c, k_layer.shape, k_layer.stride(), k_off)
    v_c = torch.as_strided(pool_c, v_layer.shape, v_layer.stride(), v_off)
    qkv_c = _f(qkv)
    _cc.qkv_rope_kv_write(qkv_c, _f(bias), _f(cos), _f(sin), _i(slot_map), k_c, v_c, page_stride, page_size,
                          n_heads, n_kv, head_dim)
    _py.qkv_rope_kv_write(qkv, bias, cos, sin, slot_map, k_layer, v_layer, page_stride, page_size, n_heads, n_kv,
                          head_dim)
    _agree(qkv[:, :n_heads * head_dim], qkv_c[:, :n_heads * head_dim], "bias + rotation (q)", qkv.dtype)
    if n_kv:
        _agree(pool, pool_c, "bias + rotation + cache write", qkv.dtype)


def attn_paged_generic(q, q_stride, out, k_layer, v_layer, page_stride, page_size, block_tables, tile_entry, tile_q0,
                       n_tiles, entry_q_start, entry_q_len, entry_ctx_start, n_heads, n_kv, head_dim, scale, window):
    _py.attn_paged_generic(q, q_stride, out, k_layer, v_layer, page_stride, page_size, block_tables, tile_entry,
                           tile_q0, n_tiles, entry_q_start, entry_q_len, entry_ctx_start, n_heads, n_kv, head_dim,
                           scale, window)
    pool = k_layer._base if k_layer._base is not None else k_layer
    pool_c = _f(pool)
    k_c = torch.as_strided(pool_c, k_layer.shape, k_layer.stride(), k_layer.storage_offset())
    v_c = torch.as_strided(pool_c, v_layer.shape, v_layer.stride(), v_layer.storage_offset())
    q_c = _f(q)
    out_c = torch.zeros((q_c.shape[0], n_heads * head_dim), dtype=torch.float32)
    _cc.attention_paged(q_c, q_c.stride(0), out_c, k_c, v_c, page_stride, page_size, _i(block_tables),
                        _i(entry_q_start), _i(entry_q_len), _i(entry_ctx_start), n_heads, n_kv, head_dim, scale, window)
    _agree(out, out_c, "paged attention", out.dtype)
    return out


def apply_penalties(logits, recent_ids, recent_counts, n_recent, rep, freq, pres):
    logits_c = _f(logits)
    _cc.apply_penalties(logits_c, _i(recent_ids), _i(recent_counts), _i(n_recent), _f(rep), _f(freq), _f(pres))
    _py.apply_penalties(logits, recent_ids, recent_counts, n_recent, rep, freq, pres)
    _agree(logits, logits_c, "penalties")
