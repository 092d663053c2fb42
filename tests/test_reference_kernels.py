"""The plain implementation against the reference's own kernels.

``tests/plain_qwen2.py`` restates the formulas of vjsingh1984/inferflux from a
reading of its source.  This file pins that reading: the reference's leaf
kernels (runtime/backends/cuda/native/cuda_kernels.cu,
runtime/backends/cuda/kernels/flash_attention.cu) are compiled unmodified for
sm_100a (``baseline/reference_kernels``) and each is compared, at tiny shapes,
with the matching function of the plain implementation.  The reference computes
in float32 and stores bfloat16, so the allowance is one bfloat16 rounding of the
result (2^-8 of the largest value) plus a little for float32 arithmetic.

The test is skipped when the reference's sources have not been fetched into
``baseline/_ref/inferflux_src`` (they are not part of this repository).
"""
from __future__ import annotations

import ctypes
import math

import pytest
import torch

import plain_qwen2 as plain

pytestmark = pytest.mark.gpu

BF16_ROUNDING = 2.0 ** -8 * 1.15


@pytest.fixture(scope="module")
def ref():
    from baseline import reference_kernels
    if reference_kernels.source_root() is None:
        pytest.skip("the reference's kernel sources are not under baseline/_ref/inferflux_src "
                    "(python -m baseline.reference_kernels fetch <reference checkout>)")
    return reference_kernels.load()


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ok(rc):
    assert rc == 0, f"the reference's wrapper returned cudaError {rc}"
    torch.cuda.synchronize()


def _bf16(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).cuda()


def _close(got, want, what, allowance=BF16_ROUNDING):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max() / want.abs().max())
    assert err <= allowance, f"{what}: {err:.3e} of the largest value"


@pytest.mark.parametrize("t,nh,nkv,hd,n_past,theta", [(9, 4, 2, 16, 0, 1e4), (5, 3, 1, 32, 37, 1e6),
                                                       (1, 7, 1, 128, 300, 1e6)])
def test_rope_split_half(ref, t, nh, nkv, hd, n_past, theta):
    q, k = _bf16((t, nh * hd), 1), _bf16((t, nkv * hd), 2)
    q0, k0 = q.clone(), k.clone()
    _ok(ref.ref_rope_neox(_p(q), _p(k), t, nh, nkv, hd, n_past, ctypes.c_float(theta), _stream()))
    pos = torch.arange(n_past, n_past + t)
    cos, sin = plain.rope_angles(pos, hd, theta, torch.float64)
    _close(q.view(t, nh, hd), plain.apply_rope_half(q0.double().cpu().view(t, nh, hd), cos, sin), "rotated q")
    _close(k.view(t, nkv, hd), plain.apply_rope_half(k0.double().cpu().view(t, nkv, hd), cos, sin), "rotated k")


@pytest.mark.parametrize("rows,hidden,eps", [(3, 64, 1e-6), (5, 96, 1e-5), (2, 80, 3e-6), (2, 3584, 1e-6)])
def test_rms_norm_and_residual_add(ref, rows, hidden, eps):
    g = torch.Generator().manual_seed(hidden)
    x = torch.randn((rows, hidden), generator=g).cuda()
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16).cuda()
    out = torch.empty((rows, hidden), dtype=torch.bfloat16, device="cuda")
    _ok(ref.ref_rms_norm_mixed(_p(x), _p(w), _p(out), rows, hidden, ctypes.c_float(eps), _stream()))
    _close(out, plain.rms_norm(x.double().cpu(), w.double().cpu(), eps), "RmsNormMixed")
    delta = _bf16((rows, hidden), 5)
    res = x.clone()
    _ok(ref.ref_residual_add_rms_norm_mixed(_p(res), _p(delta), _p(w), _p(out), rows, hidden, ctypes.c_float(eps),
                                            _stream()))
    summed = x.double().cpu() + delta.double().cpu()
    _close(res, summed, "residual after the add", 1e-6)
    _close(out, plain.rms_norm(summed, w.double().cpu(), eps), "ResidualAddRmsNormMixed")


def test_silu_mul(ref):
    gate, up = _bf16((7, 176), 3, 3.0), _bf16((7, 176), 4)
    out = torch.empty_like(gate)
    _ok(ref.ref_silu_mul(_p(gate), _p(up), _p(out), gate.numel(), _stream()))
    _close(out, plain.silu_mul(gate.double().cpu(), up.double().cpu()), "SiluMul")


def test_bias_add_triple(ref):
    rows, qd, kd = 5, 96, 32
    q, k, v = _bf16((rows, qd), 1), _bf16((rows, kd), 2), _bf16((rows, kd), 3)
    bq, bk, bv = _bf16((qd,), 4), _bf16((kd,), 5), _bf16((kd,), 6)
    want = [(x.double() + b.double()).cpu() for x, b in ((q, bq), (k, bk), (v, bv))]
    _ok(ref.ref_bias_add_triple(_p(q), _p(k), _p(v), _p(bq), _p(bk), _p(bv), rows, qd, kd, kd, _stream()))
    for got, w, name in zip((q, k, v), want, "qkv"):
        _close(got, w, f"BiasAddTriple {name}")


def test_embedding_lookup(ref):
    table = _bf16((777, 80), 9)
    ids = torch.tensor([5, 776, 0, 5, 123], dtype=torch.int32, device="cuda")
    out = torch.empty((5, 80), dtype=torch.float32, device="cuda")
    _ok(ref.ref_embedding_lookup_f32(_p(table), _p(ids), _p(out), 5, 80, _stream()))
    assert torch.equal(out.cpu().double(), plain.embed(table.double().cpu(), ids.tolist()))


def _attention_inputs(kv_len, nh, nkv, hd, seed):
    """Queries and keys with one far key made to stand out for the last
    queries, so that a wrong causal limit or kv head would show."""
    q, k, v = _bf16((kv_len, nh, hd), seed, 1.0), _bf16((kv_len, nkv, hd), seed + 1, 1.0), _bf16((kv_len, nkv, hd), seed + 2)
    k[3] = (k[3].float() * 3).to(torch.bfloat16)
    q[-1] = (k[3].repeat_interleave(nh // nkv, dim=0).float() * 0.5).to(torch.bfloat16)
    return q, k, v


# Ratios 7, 3 and 5 reach FlashAttention2TypedKernel (flash_attention.cu:432-447), which is what Qwen2.5-7B gets
# there.  Head sizes start at 64: the kernel runs next_pow2(head_dim) threads and lets thread d finish score d of a
# 64-key tile (flash_attention.cu:127-133), so with fewer than 64 threads the scores beyond the block's size are
# never written; at head size 32 and more than 32 keys its output differs from the formula by a quarter.
@pytest.mark.parametrize("nh,nkv,hd", [(7, 1, 64), (6, 2, 64), (5, 1, 80), (14, 2, 128)])
@pytest.mark.parametrize("q_len,kv_len", [(1, 77), (33, 100), (70, 70)])
def test_flash_attention2(ref, nh, nkv, hd, q_len, kv_len):
    q, k, v = _attention_inputs(kv_len, nh, nkv, hd, 11)
    scale = 1.0 / math.sqrt(hd)
    want = plain.causal_gqa_attention(q.double().cpu(), k.double().cpu(), v.double().cpu(), scale)[kv_len - q_len:]
    q_new = q[kv_len - q_len:].contiguous()
    out = torch.empty_like(q_new)
    _ok(ref.ref_flash_attention2(_p(q_new), _p(k), _p(v), _p(out), 1, q_len, kv_len, nh, nkv, hd,
                                 ctypes.c_float(scale), 1, _stream()))
    _close(out, want, "FlashAttention2Typed")


@pytest.mark.parametrize("nh,nkv,hd", [(7, 1, 64), (6, 2, 64), (5, 1, 80), (28, 4, 128)])
def test_flash_decode_multi_seq(ref, nh, nkv, hd):
    lens = [1, 64, 65, 200]
    scale = 1.0 / math.sqrt(hd)
    qs, ks, vs, wants = [], [], [], []
    for i, n in enumerate(lens):
        q, k, v = _attention_inputs(max(n, 4), nh, nkv, hd, 20 + 3 * i)
        q, k, v = q[:n], k[:n].contiguous(), v[:n].contiguous()
        wants.append(plain.causal_gqa_attention(q.double().cpu(), k.double().cpu(), v.double().cpu(), scale)[-1])
        qs.append(q[-1]), ks.append(k), vs.append(v)
    q = torch.stack(qs).contiguous()
    out = torch.empty_like(q)
    k_ptrs = torch.tensor([k.data_ptr() for k in ks], dtype=torch.int64, device="cuda")
    v_ptrs = torch.tensor([v.data_ptr() for v in vs], dtype=torch.int64, device="cuda")
    kv_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    _ok(ref.ref_flash_decode_multi_seq(_p(q), _p(k_ptrs), _p(v_ptrs), _p(out), _p(kv_lens), len(lens), nh, nkv, hd,
                                       ctypes.c_float(scale), _stream()))
    _close(out, torch.stack(wants), "FlashDecodeMultiSeq")
