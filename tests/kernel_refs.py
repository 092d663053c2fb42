"""Plain PyTorch float32 references of the kernels, one function per kernel
with the kernel wrapper's signature (``inferflux_b200.kernels.ops``).  They run
on whatever device their operands are on, loop where the kernel is clever, and
are only used by tests.
"""
from __future__ import annotations

import math

import torch


def embed_gather(table, ids, out):
    out.copy_(table[ids.long()].float())
    return out


def add_rmsnorm(residual, delta, weight, eps, out, rows=None, n_partials=1):
    r = residual
    if delta is not None:
        d = delta.float().sum(0) if n_partials > 1 else delta.float()
        r = residual + d
        if rows is None:
            residual.copy_(r)
    if rows is not None:
        r = r[rows.long()]
    if out is not None:
        y = r * torch.rsqrt((r * r).mean(-1, keepdim=True) + eps) * weight
        out.copy_(y.to(out.dtype))
    return out


def swiglu(gate_up, out):
    i = gate_up.shape[1] // 2
    g, u = gate_up[:, :i].float(), gate_up[:, i:].float()
    out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))
    return out


def convert(src, dst):
    dst.copy_(src.to(dst.dtype))
    return dst


def rope_table(positions, inv_freq, cos, sin):
    a = positions.double()[:, None] * inv_freq[None, :]
    cos.copy_(torch.cos(a).float())
    sin.copy_(torch.sin(a).float())


def qkv_rope_kv_write(qkv, bias, cos, sin, slot_map, k_layer, v_layer, page_stride, page_size,
                      n_heads, n_kv, head_dim):
    n = qkv.shape[0]
    x = qkv.float()
    if bias is not None:
        x = x + bias
    half = cos.shape[1]
    heads = x.view(n, n_heads + 2 * n_kv, head_dim)
    rot = heads[:, :n_heads + n_kv]
    x0, x1, rest = rot[..., :half], rot[..., half:2 * half], rot[..., 2 * half:]
    c, s = cos[:, None, :], sin[:, None, :]
    rotated = torch.cat([x0 * c - x1 * s, x0 * s + x1 * c, rest], -1).to(qkv.dtype)
    qkv.view(n, n_heads + 2 * n_kv, head_dim)[:, :n_heads] = rotated[:, :n_heads]
    if n_kv:
        # k_layer / v_layer are views [n_kv, page_size, head_dim] of page 0; pages lie page_stride apart
        kflat = _pool_view(k_layer, page_stride)
        vflat = _pool_view(v_layer, page_stride)
        for t in range(n):
            slot = int(slot_map[t])
            if slot < 0:
                continue
            page, off = slot // page_size, slot % page_size
            kflat[page][:, off, :] = rotated[t, n_heads:]
            vflat[page][:, off, :] = heads[t, n_heads + n_kv:].to(qkv.dtype)


class _PoolView:
    """Indexes pages of a layer given the view of page 0 and the page stride."""

    def __init__(self, layer0, page_stride):
        self.layer0, self.page_stride = layer0, page_stride

    def __getitem__(self, page):
        l0 = self.layer0
        return torch.as_strided(l0, l0.shape, l0.stride(), l0.storage_offset() + page * self.page_stride)


def _pool_view(layer0, page_stride):
    return _PoolView(layer0, page_stride)


def gemm_f32(a, w, bias, out):
    y = a.float() @ w.float().T
    if bias is not None:
        y = y + bias
    out.copy_(y)
    return out


def gemv_bf16(x, w, bias, out, swiglu=False, k_splits=1):
    if k_splits > 1:
        k = x.shape[1]
        chunks = (k + 31) // 32
        per = (chunks + k_splits - 1) // k_splits
        for s in range(k_splits):
            lo, hi = min(k, s * per * 32), min(k, (s + 1) * per * 32)
            out[s] = x[:, lo:hi].float() @ w[:, lo:hi].float().T
        if bias is not None:
            out[0] += bias
        return out
    y = x.float() @ w.float().T
    if swiglu:
        n = out.shape[1]
        g, u = y[:, :n], y[:, n:]
        y = g / (1.0 + torch.exp(-g)) * u
    elif bias is not None:
        y = y + bias
    out.copy_(y.to(out.dtype))
    return out


def attn_paged_generic(q, q_stride, out, k_layer, v_layer, page_stride, page_size, block_tables,
                       tile_entry, tile_q0, n_tiles, entry_q_start, entry_q_len, entry_ctx_start,
                       n_heads, n_kv, head_dim, scale, window):
    """Per entry: gather its keys and values from the pages, then plain causal
    (windowed) softmax attention per head."""
    kp, vp = _pool_view(k_layer, page_stride), _pool_view(v_layer, page_stride)
    ratio = n_heads // n_kv
    for e in range(entry_q_start.numel()):
        qs, ql, cs = int(entry_q_start[e]), int(entry_q_len[e]), int(entry_ctx_start[e])
        total = cs + ql
        keys = torch.zeros(total, n_kv, head_dim)
        vals = torch.zeros(total, n_kv, head_dim)
        for pos in range(total):
            page = int(block_tables[e, pos // page_size])
            if page >= 0:
                keys[pos] = kp[page][:, pos % page_size, :].float().cpu()
                vals[pos] = vp[page][:, pos % page_size, :].float().cpu()
        qrows = q[qs:qs + ql, :n_heads * head_dim].float().cpu().view(ql, n_heads, head_dim)
        for i in range(ql):
            p = cs + i
            lo = max(0, p - window + 1) if window > 0 else 0
            for h in range(n_heads):
                kh = h // ratio
                s = (keys[lo:p + 1, kh] @ qrows[i, h]) * scale
                pr = torch.softmax(s, 0)
                out[qs + i, h * head_dim:(h + 1) * head_dim] = (pr @ vals[lo:p + 1, kh]).to(out.dtype)
    return out


def argmax(logits, out):
    out[:logits.shape[0]] = torch.argmax(logits, dim=-1).int()   # torch returns the first maximum on CPU
    return out


def apply_penalties(logits, recent_ids, recent_counts, n_recent, rep, freq, pres):
    for r in range(logits.shape[0]):
        for k in range(int(n_recent[r])):
            t, c = int(recent_ids[r, k]), int(recent_counts[r, k])
            v = logits[r, t]
            v = v / rep[r] if v > 0 else v * rep[r]
            v = v - freq[r] * c
            if c > 0:
                v = v - pres[r]
            logits[r, t] = v


def uniform01(seed: int, counter: int) -> float:
    """The kernel's counter-based uniform (a 64-bit mixing function), 24 bits."""
    mask = (1 << 64) - 1

    def mix(z):
        z = (z + 0x9E3779B97F4A7C15) & mask
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        return z ^ (z >> 31)
    x = mix(mix(seed & mask) ^ ((counter * 0xD1342543DE82EF95 + 0x632BE59BD9B4E019) & mask))
    return (x >> 40) / 16777216.0
