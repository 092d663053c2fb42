"""Each CUDA kernel alone against its two references, the plain PyTorch one
(tests/kernel_refs.py) and the host-side C++ one (csrc/host_reference), which
tests/checked_refs.py also holds against each other, at sizes other than the
engine's test models: row
lengths that are no power of two, head sizes in steps of 16, odd head counts
and group ratios, page sizes 4 to 64.  Where random inputs would hide a fault
(one far key among hundreds, a window's edge, a page border) the inputs are
made so that it shows."""
from __future__ import annotations

import math

import pytest
import torch

import checked_refs as ref
from inferflux_b200.kernels import host_reference as host

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from inferflux_b200.kernels import ops as o
    return o


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


def _close(got, want, tol, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol}"


# ------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab,hidden", [(37, 24), (1000, 100), (513, 3584)])
def test_embed_gather(ops, dtype, vocab, hidden):
    table = _rand((vocab, hidden), dtype, 1)
    ids = torch.tensor([0, vocab - 1, 5, 5, vocab // 2], dtype=torch.int32, device=DEV)
    out = torch.empty((5, hidden), dtype=torch.float32, device=DEV)
    ops.embed_gather(table, ids, out)
    assert torch.equal(out.cpu(), table.cpu()[ids.cpu().long()].float())
    assert torch.equal(out.cpu(), host.embed_gather(table.float().cpu(), ids.cpu(), torch.empty((5, hidden))))


@pytest.mark.parametrize("hidden", [24, 100, 3584, 5120 + 8])
@pytest.mark.parametrize("ddt,odt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.float32, torch.bfloat16)])
def test_add_rmsnorm(ops, hidden, ddt, odt):
    n = 7
    res = _rand((n, hidden), torch.float32, 2)
    delta = _rand((n, hidden), ddt, 3)
    w = _rand((hidden,), torch.float32, 4) + 1.0
    res_ref, out_ref = res.clone().cpu(), torch.empty((n, hidden), dtype=odt)
    ref.add_rmsnorm(res_ref, delta.cpu(), w.cpu(), 1e-5, out_ref)
    out = torch.empty((n, hidden), dtype=odt, device=DEV)
    ops.add_rmsnorm(res, delta, w, 1e-5, out)
    _close(res, res_ref, 1e-6, "residual")
    _close(out, out_ref, 1e-5 if odt == torch.float32 else 8e-3, "normed")
    # gather mode: listed rows only, a row listed twice, the residual untouched
    rows = torch.tensor([6, 0, 6], dtype=torch.int32, device=DEV)
    before = res.clone()
    out2 = torch.empty((3, hidden), dtype=odt, device=DEV)
    ops.add_rmsnorm(res, delta, w, 1e-5, out2, rows)
    assert torch.equal(res, before)
    out2_ref = torch.empty((3, hidden), dtype=odt)
    ref.add_rmsnorm(before.cpu(), delta.cpu(), w.cpu(), 1e-5, out2_ref, rows.cpu())
    _close(out2, out2_ref, 1e-5 if odt == torch.float32 else 8e-3, "gathered")
    # no delta
    out3 = torch.empty((n, hidden), dtype=odt, device=DEV)
    ops.add_rmsnorm(res, None, w, 1e-5, out3)
    out3_ref = torch.empty((n, hidden), dtype=odt)
    ref.add_rmsnorm(before.cpu(), None, w.cpu(), 1e-5, out3_ref)
    _close(out3, out3_ref, 1e-5 if odt == torch.float32 else 8e-3, "no delta")


@pytest.mark.parametrize("hidden", [24, 100, 1024, 2048, 3584, 5120, 8192])
@pytest.mark.parametrize("parts", [1, 5])
def test_add_rmsnorm_same_bits_whatever_the_number_of_rows(ops, hidden, parts):
    """A step of a few rows spreads a row over up to 1,024 threads, a step of many rows gives it 256; the squares
    are added in the same order in both, so a row's residual and normed values are the same bit for bit."""
    n_small, n_big = 3, 100
    res = _rand((n_big, hidden), torch.float32, 50)
    delta = _rand((parts, n_big, hidden), torch.float32, 51)
    w = _rand((hidden,), torch.float32, 52) + 1.0
    big_res, small_res = res.clone(), res[:n_small].clone()
    big_out = torch.empty((n_big, hidden), dtype=torch.float32, device=DEV)
    small_out = torch.empty((n_small, hidden), dtype=torch.float32, device=DEV)
    ops.add_rmsnorm(big_res, delta if parts > 1 else delta[0], w, 1e-6, big_out, n_partials=parts)
    small_delta = delta[:, :n_small].contiguous()
    ops.add_rmsnorm(small_res, small_delta if parts > 1 else small_delta[0], w, 1e-6, small_out, n_partials=parts)
    assert torch.equal(small_res, big_res[:n_small]) and torch.equal(small_out, big_out[:n_small])


def test_add_rmsnorm_partials(ops):
    n, hidden, parts = 5, 200, 3
    res = _rand((n, hidden), torch.float32, 5)
    delta = _rand((parts, n, hidden), torch.float32, 6)
    w = torch.ones(hidden, device=DEV)
    want = res.cpu() + delta.cpu().sum(0)
    out = torch.empty((n, hidden), dtype=torch.float32, device=DEV)
    ops.add_rmsnorm(res, delta, w, 1e-6, out, n_partials=parts)
    _close(res, want, 1e-6, "partials")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m,inter", [(1, 7), (5, 176), (33, 18944)])
def test_swiglu(ops, dtype, m, inter):
    gu = _rand((m, 2 * inter), dtype, 7, 2.0)
    out = torch.empty((m, inter), dtype=dtype, device=DEV)
    ops.swiglu(gu, out)
    want = torch.empty((m, inter), dtype=dtype)
    ref.swiglu(gu.cpu(), want)
    _close(out, want, 1e-6 if dtype == torch.float32 else 8e-3, "swiglu")


@pytest.mark.parametrize("m,n,k", [(1, 5, 3), (7, 100, 96), (65, 130, 257), (128, 64, 64), (3, 1000, 80)])
def test_gemm_f32(ops, m, n, k):
    a, w, b = _rand((m, k), torch.float32, 8), _rand((n, k), torch.float32, 9), _rand((n,), torch.float32, 10)
    out = torch.empty((m, n), dtype=torch.float32, device=DEV)
    ops.gemm_f32(a, w, b, out)
    want = a.double().cpu() @ w.double().cpu().T + b.double().cpu()
    _close(out, want, 2e-6, "gemm_f32")
    _close(out, host.gemm(a.cpu(), w.cpu(), b.cpu(), torch.empty((m, n))), 2e-6, "gemm_f32 against the C++ loops")
    # a row's result does not depend on the other rows (bitwise)
    one = torch.empty((1, n), dtype=torch.float32, device=DEV)
    ops.gemm_f32(a[m - 1:m], w, b, one)
    assert torch.equal(one[0], out[m - 1])


def test_gemm_f32_is_true_float32(ops):
    """Values that a reduced-precision (tf32, 10-bit mantissa) product would lose."""
    k = 64
    a = torch.full((1, k), 1.0 + 2.0 ** -12, device=DEV)
    w = torch.full((1, k), 1.0 + 2.0 ** -12, device=DEV)
    out = torch.empty((1, 1), device=DEV)
    ops.gemm_f32(a, w, None, out)
    want = k * (1.0 + 2.0 ** -12) ** 2
    assert abs(float(out) - want) / want < 1e-6


@pytest.mark.parametrize("m", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(16, 32), (100, 96), (1000, 64), (4608, 3584), (37, 200), (152064, 128), (48, 2312)])
@pytest.mark.parametrize("odt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("impl", ["gemv_bf16"])
def test_gemv_bf16(ops, m, n, k, odt, impl):
    if n > 10000 and m not in (1, 9):
        pytest.skip("large case at two row counts only")
    gemv = getattr(ops, impl)
    x, w, b = _rand((m, k), torch.bfloat16, 40), _rand((n, k), torch.bfloat16, 41, 0.1), _rand((n,), torch.float32, 42)
    out = torch.empty((m, n), dtype=odt, device=DEV)
    gemv(x, w, b, out)
    want = x.double().cpu() @ w.double().cpu().T + b.double().cpu()
    _close(out, want, 1e-5 if odt == torch.float32 else 6e-3, "gemv")
    # a token's result does not depend on the other rows (bitwise)
    one = torch.empty((1, n), dtype=odt, device=DEV)
    gemv(x[m - 1:m], w, b, one)
    assert torch.equal(one[0], out[m - 1])
    ops.check_device_errors(DEV)


@pytest.mark.parametrize("impl", ["gemv_bf16"])
@pytest.mark.parametrize("m,n,k,splits", [(1, 3584, 18944, 3), (8, 3584, 3584, 3), (13, 100, 96, 2), (16, 40, 4096, 4),
                                          (5, 64, 64, 4)])
def test_gemv_split_k(ops, m, n, k, splits, impl):
    x, w, b = _rand((m, k), torch.bfloat16, 45), _rand((n, k), torch.bfloat16, 46, 0.1), _rand((n,), torch.float32, 47)
    out = torch.empty((splits, m, n), dtype=torch.float32, device=DEV)
    getattr(ops, impl)(x, w, b, out, k_splits=splits)
    want = x.double().cpu() @ w.double().cpu().T + b.double().cpu()
    _close(out.sum(0), want, 1e-5, "gemv split-K")
    ops.check_device_errors(DEV)


@pytest.mark.parametrize("impl", ["gemv_bf16"])
@pytest.mark.parametrize("m", [1, 8, 13, 16])
@pytest.mark.parametrize("inter,k", [(8, 32), (176, 64), (100, 96), (18944, 3584), (5, 40)])
def test_gemv_swiglu(ops, m, inter, k, impl):
    x, w = _rand((m, k), torch.bfloat16, 43), _rand((2 * inter, k), torch.bfloat16, 44, 0.2)
    out = torch.empty((m, inter), dtype=torch.bfloat16, device=DEV)
    getattr(ops, impl)(x, w, None, out, swiglu=True)
    want = torch.empty((m, inter), dtype=torch.float32)
    ref.gemv_bf16(x.cpu(), w.cpu(), None, want, swiglu=True)
    _close(out, want, 6e-3, "gemv swiglu")


# ----------------------------------------------------------------------- rotary
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rot,ps", [(4, 2, 16, 16, 16), (3, 1, 32, 32, 4), (10, 2, 48, 24, 8),
                                              (28, 4, 128, 128, 16), (5, 5, 80, 80, 64), (2, 0, 64, 64, 16)])
@pytest.mark.parametrize("n", [19, 301])        # 301 tokens: the kernel that takes several tokens a block
def test_rope_and_kv_write(ops, dtype, nh, nkv, hd, rot, ps, n):
    pages, layers = (n + ps - 1) // ps + 7, 2
    first = [0, 1, 2, 3, 500, 501, 4095, 31, 32, 33, 7, 8, 9, 10, 11, 12, 13, 14, 15]
    positions = torch.tensor((first + list(range(600, 600 + n)))[:n], dtype=torch.int32, device=DEV)
    inv = torch.pow(torch.tensor(1e6, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot).to(DEV)
    cos = torch.empty((n, rot // 2), dtype=torch.float32, device=DEV)
    sin = torch.empty_like(cos)
    ops.rope_table(positions, inv, cos, sin)
    ang = positions.double().cpu()[:, None] * inv.cpu()[None, :]
    _close(cos, torch.cos(ang), 1e-6, "cos")
    _close(sin, torch.sin(ang), 1e-6, "sin")
    width = (nh + 2 * nkv) * hd
    qkv = _rand((n, width), dtype, 11)
    bias = _rand((width,), torch.float32, 12)
    pool = torch.zeros((pages, layers, 2, max(nkv, 1), ps, hd), dtype=dtype, device=DEV)
    slots = torch.randperm(pages * ps, generator=torch.Generator().manual_seed(1))[:n].int().to(DEV)
    slots[3] = -1                                            # not stored
    qkv_ref, pool_ref = qkv.clone().cpu(), pool.clone().cpu()
    ref.qkv_rope_kv_write(qkv_ref, bias.cpu(), cos.cpu(), sin.cpu(), slots.cpu(), pool_ref[0, 1, 0], pool_ref[0, 1, 1],
                          pool_ref.stride(0), ps, nh, nkv, hd)
    ops.qkv_rope_kv_write(qkv, bias, cos, sin, slots if nkv else None, pool[0, 1, 0] if nkv else None,
                          pool[0, 1, 1] if nkv else None, pool.stride(0), ps, nh, nkv, hd)
    tol = 1e-6 if dtype == torch.float32 else 8e-3
    _close(qkv[:, :nh * hd], qkv_ref[:, :nh * hd], tol, "q")
    if nkv:
        _close(pool, pool_ref, tol, "cache")
        assert float(pool[:, 0].abs().max()) == 0.0          # the other layer's pages are untouched


# -------------------------------------------------------------------- attention
def _attention_case(ops, dtype, nh, nkv, hd, ps, window, entries, seed, peaked, fast, umma=False):
    """entries: list of (cached tokens, new tokens).  Builds a paged cache with
    scattered pages, runs the kernel(s) and the reference."""
    from inferflux_b200.parts.attention import CHUNK_TILE, QUERY_TILE
    g = torch.Generator().manual_seed(seed)
    n = sum(q for _, q in entries)
    total_pages = sum((c + q + ps - 1) // ps for c, q in entries) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()
    pool = torch.zeros((total_pages, 1, 2, nkv, ps, hd), dtype=dtype)
    width = max((c + q + ps - 1) // ps for c, q in entries)
    bt = torch.full((len(entries), width), -1, dtype=torch.int32)
    q = torch.randn((n, nh * hd), generator=g)
    q_start, q_len, ctx_start, tiles, ctiles, decs = [], [], [], [], [], []
    row = 0
    for e, (c, ql) in enumerate(entries):
        nblocks = (c + ql + ps - 1) // ps
        for b in range(nblocks):
            bt[e, b] = perm.pop()
        keys = torch.randn((c + ql, nkv, hd), generator=g)
        vals = torch.randn((c + ql, nkv, hd), generator=g)
        if peaked:
            # one far key per (query row, kv head) dominates: the output is close to that key's value
            for i in range(ql):
                pos = c + i
                lo = max(0, pos - window + 1) if window else 0
                far = lo if i % 2 == 0 else (lo + pos) // 2
                for h in range(nh):
                    kh = h // (nh // nkv)
                    if i % 3 == h % 3:
                        q[row + i, h * hd:(h + 1) * hd] = keys[far, kh] * 3.0
        if window:
            first_needed = max(0, c - window + 1) // ps          # blocks before it were given back
            for b in range(first_needed):
                bt[e, b] = -1
        for pos in range(c + ql):
            page = int(bt[e, pos // ps])
            if page >= 0:
                pool[page, 0, 0, :, pos % ps] = keys[pos].to(dtype)
                pool[page, 0, 1, :, pos % ps] = vals[pos].to(dtype)
        q_start.append(row), q_len.append(ql), ctx_start.append(c)
        tiles += [(e, q0) for q0 in range(0, ql, QUERY_TILE)]
        if ql == 1:
            decs.append(e)
        else:
            ctiles += [(e, q0) for q0 in range(0, ql, CHUNK_TILE)]
        row += ql
    q = q.to(dtype)
    it = lambda v: torch.tensor(v, dtype=torch.int32)
    meta = dict(q_start=it(q_start), q_len=it(q_len), ctx_start=it(ctx_start))
    scale = 1.0 / math.sqrt(hd)
    want = torch.zeros((n, nh * hd), dtype=torch.float32)
    poolf = pool.float()
    ref.attn_paged_generic(q.float(), nh * hd, want, poolf[0, 0, 0], poolf[0, 0, 1], poolf.stride(0), ps, bt,
                           None, None, 0, meta["q_start"], meta["q_len"], meta["ctx_start"], nh, nkv, hd, scale,
                           window or 0)
    qd, poold, btd = q.to(DEV), pool.to(DEV), bt.to(DEV)
    md = {k: v.to(DEV) for k, v in meta.items()}
    out = torch.zeros((n, nh * hd), dtype=dtype, device=DEV)
    args = (poold[0, 0, 0], poold[0, 0, 1], poold.stride(0), ps, btd)
    if not fast:
        te, tq = it([t[0] for t in tiles]).to(DEV), it([t[1] for t in tiles]).to(DEV)
        ops.attn_paged_generic(qd, nh * hd, out, *args, te, tq, len(tiles), md["q_start"], md["q_len"], md["ctx_start"],
                               nh, nkv, hd, scale, window or 0)
    else:
        if ctiles and umma:
            for tile_rows, parts in ((ops.UMMA_ATTENTION_TILE, (1, 2, 5)), (ops.UMMA_ATTENTION_TILE // 2, (1, 3))):
                utiles = [(e, q0) for e, (c, ql) in enumerate(entries) if ql > 1 for q0 in range(0, ql, tile_rows)]
                te, tq = it([t[0] for t in utiles]).to(DEV), it([t[1] for t in utiles]).to(DEV)
                for splits in parts:                      # the keys of a query tile in one part and cut into parts
                    out_u = out.clone()
                    ops.attn_prefill_umma(qd, nh * hd, out_u, *args, te, tq, len(utiles), md["q_start"], md["q_len"],
                                          md["ctx_start"], nh, nkv, hd, scale, window or 0, splits, tile_rows)
                    ops.check_device_errors(DEV)
                    rows = [r for e, (c, ql) in enumerate(entries) if ql > 1 for r in range(q_start[e], q_start[e] + ql)]
                    _close(out_u[rows], want[rows], 1.5e-2, f"prompt attention, tiles of {tile_rows}, keys in {splits} parts")
            out = out_u
        elif ctiles:
            te, tq = it([t[0] for t in ctiles]).to(DEV), it([t[1] for t in ctiles]).to(DEV)
            ops.attn_prefill_bf16(qd, nh * hd, out, *args, te, tq, len(ctiles), md["q_start"], md["q_len"],
                                  md["ctx_start"], nh, nkv, hd, scale, window or 0)
        if decs:
            for splits in ([1, 3, 8] if len(entries) < 6 else [4]):
                out_d = out.clone()
                po = torch.empty(len(decs) * nh * splits * hd, dtype=torch.float32, device=DEV)
                pm = torch.empty(len(decs) * nh * splits * 2, dtype=torch.float32, device=DEV)
                ops.attn_decode_bf16(qd, nh * hd, out_d, *args, it(decs).to(DEV), len(decs), md["q_start"], md["q_len"],
                                     md["ctx_start"], po, pm, nh, nkv, hd, scale, window or 0, splits)
                _close(out_d, want, 1.5e-2, f"decode attention, {splits} splits")
            # the kernel that shares the tiles of all entries out evenly, with exact and with loose bounds on the contexts
            longest = max(min(c + 1, window) if window else c + 1 for c, ql in entries if ql == 1)
            for bound in (longest, 4 * longest + 100):
                pieces = ops.attn_decode_pieces(nh, nkv, hd, bound)
                out_e = out.clone()
                po = torch.full((len(decs) * nh * pieces * hd,), float("nan"), dtype=torch.float32, device=DEV)
                pm = torch.full((len(decs) * nh * pieces * 2,), float("nan"), dtype=torch.float32, device=DEV)
                pc = torch.full((len(decs) * nh,), -7, dtype=torch.int32, device=DEV)
                ops.attn_decode_even_bf16(qd, out_e, *args, it(decs).to(DEV), len(decs), md["q_start"], md["q_len"],
                                          md["ctx_start"], po, pm, pc, nh, nkv, hd, scale, window or 0, pieces)
                ops.check_device_errors(DEV)
                _close(out_e, want, 1.5e-2, f"decode attention, tiles shared out evenly, {pieces} pieces")
            out = out_d
    _close(out, want, 2e-5 if dtype == torch.float32 else 1.5e-2, "attention")
    return out.float().cpu(), want


MIXED = [(0, 5), (37, 1), (100, 70), (0, 130), (255, 1), (16, 16), (15, 2), (300, 1), (63, 65)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(4, 2, 16, 16, None), (3, 1, 32, 4, 24), (10, 2, 48, 8, None),
                                                 (7, 1, 128, 16, 100), (6, 3, 80, 64, None), (2, 2, 256, 16, 33)])
@pytest.mark.parametrize("peaked", [False, True])
def test_attention_generic(ops, dtype, nh, nkv, hd, ps, window, peaked):
    _attention_case(ops, dtype, nh, nkv, hd, ps, window, MIXED, 20, peaked, fast=False)


@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(28, 4, 128, 16, None), (16, 2, 128, 16, None), (5, 1, 64, 8, None),
                                                 (3, 3, 64, 32, 40), (40, 2, 128, 16, None), (14, 2, 128, 4, 129),
                                                 (8, 8, 128, 64, None)])
@pytest.mark.parametrize("peaked", [False, True])
def test_attention_tensor_core(ops, nh, nkv, hd, ps, window, peaked):
    _attention_case(ops, torch.bfloat16, nh, nkv, hd, ps, window, MIXED, 21, peaked, fast=True)


@pytest.mark.parametrize("nh,nkv,ps,window", [(28, 4, 16, None), (3, 1, 4, 129), (8, 8, 64, None), (2, 1, 16, 40)])
@pytest.mark.parametrize("peaked", [False, True])
def test_attention_tcgen05_prompt_portions(ops, nh, nkv, ps, window, peaked):
    """The tcgen05 / tensor-memory kernel for prompt portions (head size 128), beside the decode kernel."""
    entries = MIXED + [(0, 300), (200, 129), (5, 128), (700, 260)]
    _attention_case(ops, torch.bfloat16, nh, nkv, 128, ps, window, entries, 23, peaked, fast=True, umma=True)


def test_attention_long_context_far_key(ops):
    """4,000 cached keys; the query matches key 3 only: a fault in an early page shows."""
    for fast, umma in ((False, False), (True, False), (True, True)):
        _attention_case(ops, torch.bfloat16, 4, 1, 128, 16, None, [(4000, 1), (3990, 40)], 22, True, fast, umma)
    # the tcgen05 kernel over 9,000 keys: two query tiles a block and one tile on both halves, 140 key tiles each;
    # and a window of 1,000 keys over pages of 64 (the first pages given back)
    _attention_case(ops, torch.bfloat16, 2, 1, 128, 16, None, [(9000, 1), (8700, 300)], 24, True, True, True)
    _attention_case(ops, torch.bfloat16, 3, 3, 128, 64, 1000, [(5000, 290), (4990, 1)], 25, True, True, True)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_attention_tensor_core_random_steps(ops, seed):
    """Ten steps drawn at random (heads, groups, page size, window, up to five entries of single tokens and
    portions behind contexts of up to 2,500 tokens): the tcgen05 kernel at both tile heights and with the keys
    in parts, and the decode kernels, against the reference."""
    import random
    rnd = random.Random(seed)
    done = 0
    while done < 10:
        nkv, ratio = rnd.choice([1, 2, 3, 4]), rnd.choice([1, 2, 5, 7])
        ps, window = rnd.choice([4, 8, 16, 32, 64, 128]), rnd.choice([None, None, 40, 129, 300, 1000])
        entries = [(rnd.choice([0, 0, 1, 17, 63, 64, 100, 255, 256, 300, 700, 1500, 2500]),
                    rnd.choice([1, 2, 5, 16, 65, 127, 128, 129, 200, 255, 256, 257, 300, 400, 513]))
                   for _ in range(rnd.randint(1, 5))]
        if sum(c + q for c, q in entries) > 5000:
            continue
        _attention_case(ops, torch.bfloat16, nkv * ratio, nkv, 128, ps, window, entries, rnd.randrange(10 ** 6),
                        rnd.random() < 0.5, True, True)
        ops.check_device_errors(DEV)
        done += 1


@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(28, 4, 128, 16, None), (5, 1, 64, 8, None), (40, 2, 128, 16, None),
                                                 (14, 2, 128, 4, 129), (3, 3, 64, 32, 40)])
@pytest.mark.parametrize("n_partials", [0, 1, 3])
@pytest.mark.parametrize("own_key_stands_out", [False, True])
def test_decode_attention_prepares_its_own_qkv(ops, nh, nkv, hd, ps, window, n_partials, own_key_stands_out):
    """A step of single tokens: the decode kernel that adds the bias, rotates and writes the cache itself gives
    bit for bit what the separate kernel followed by the plain decode kernel gives (output and cache), for
    contexts that end at every place of a page, with the product as bfloat16 rows and as float32 partial sums.
    In the second variant each token's own key is the one that counts: a key written late or elsewhere shows."""
    g = torch.Generator().manual_seed(70)
    cached = [0, 1, 15, 16, 17, 63, 64, 255, 300, 129]
    n, width, ratio = len(cached), (nh + 2 * nkv) * hd, nh // nkv
    pages = sum((c + 1 + ps - 1) // ps for c in cached) + 2
    perm = torch.randperm(pages, generator=g).tolist()
    pool = torch.zeros((pages, 1, 2, nkv, ps, hd), dtype=torch.bfloat16)
    bt = torch.full((n, max((c + 1 + ps - 1) // ps for c in cached)), -1, dtype=torch.int32)
    slots = []
    for e, c in enumerate(cached):
        for b in range((c + 1 + ps - 1) // ps):
            bt[e, b] = perm.pop()
        first_needed = max(0, c - window + 1) // ps if window else 0
        for pos in range(c):
            if pos // ps >= first_needed:
                pool[int(bt[e, pos // ps]), 0, :, :, pos % ps] = torch.randn((2, nkv, hd), generator=g).to(torch.bfloat16)
        slots.append(int(bt[e, c // ps]) * ps + c % ps)
        bt[e, :first_needed] = -1
    bias = torch.randn((width,), generator=g) * 0.5
    prod = torch.randn((n, width), generator=g)
    if own_key_stands_out:                                      # q + bias = 3 (k + bias) for every head of the group
        for h in range(nh):
            ksl = slice((nh + h // ratio) * hd, (nh + h // ratio + 1) * hd)
            prod[:, h * hd:(h + 1) * hd] = 3.0 * (prod[:, ksl] + bias[ksl]) - bias[h * hd:(h + 1) * hd]
    if n_partials:
        parts = torch.randn((n_partials, n, width), generator=g)
        parts[0] = prod - parts[1:].sum(0)
        parts = parts.to(DEV)
    else:
        parts = None
    ang = torch.randn((n, hd // 2), generator=g) * 3.0
    cos, sin = torch.cos(ang).to(DEV), torch.sin(ang).to(DEV)
    it = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    meta = (it(list(range(n))), n, it(list(range(n))), it([1] * n), it(cached))
    biasd, btd, slotd = bias.to(DEV), bt.to(DEV), it(slots)
    scale = 1.0 / math.sqrt(hd)
    for splits in (1, 3, 8):
        po = torch.empty(n * nh * splits * hd, dtype=torch.float32, device=DEV)
        pm = torch.empty(n * nh * splits * 2, dtype=torch.float32, device=DEV)
        # the separate kernels
        pool_a, qkv_a = pool.to(DEV), prod.to(torch.bfloat16).to(DEV)
        out_a = torch.zeros((n, nh * hd), dtype=torch.bfloat16, device=DEV)
        ops.qkv_rope_kv_write(qkv_a, biasd, cos, sin, slotd, pool_a[0, 0, 0], pool_a[0, 0, 1], pool_a.stride(0), ps,
                              nh, nkv, hd, parts)
        ops.attn_decode_bf16(qkv_a, width, out_a, pool_a[0, 0, 0], pool_a[0, 0, 1], pool_a.stride(0), ps, btd, *meta,
                             po, pm, nh, nkv, hd, scale, window or 0, splits)
        # the one kernel
        pool_b, qkv_b = pool.to(DEV), prod.to(torch.bfloat16).to(DEV)
        out_b = torch.zeros((n, nh * hd), dtype=torch.bfloat16, device=DEV)
        ops.attn_decode_prep_bf16(qkv_b, biasd, cos, sin, slotd, parts, out_b, pool_b[0, 0, 0], pool_b[0, 0, 1],
                                  pool_b.stride(0), ps, btd, *meta, po, pm, nh, nkv, hd, scale, window or 0, splits)
        assert torch.equal(pool_a, pool_b), f"{splits} splits: the caches differ"
        assert torch.equal(out_a, out_b), f"{splits} splits: the outputs differ"
        # and both against the plain attention over the cache they wrote
        want = torch.zeros((n, nh * hd), dtype=torch.float32)
        poolf = pool_b.float().cpu()
        ref.attn_paged_generic(qkv_a[:, :nh * hd].float().cpu().contiguous(), nh * hd, want, poolf[0, 0, 0], poolf[0, 0, 1],
                               poolf.stride(0), ps, bt, None, None, 0, meta[2].cpu(), meta[3].cpu(), meta[4].cpu(),
                               nh, nkv, hd, scale, window or 0)
        _close(out_b, want, 1.5e-2, f"decode attention that prepares q, k, v; {splits} splits")
        if own_key_stands_out:
            v_new = torch.stack([pool_b[s // ps, 0, 1, :, s % ps] for s in slots]).float().cpu()      # [n, nkv, hd]
            got = out_b.float().cpu().view(n, nkv, ratio, hd)
            assert (got - v_new[:, :, None, :]).abs().max() < 0.05, "the output is not the token's own value"


@pytest.mark.parametrize("m,nh,nkv,k,ps,with_bias", [(300, 3, 1, 200, 16, True), (513, 5, 2, 1096, 64, False),
                                                     (2048, 28, 4, 3584, 16, True), (70, 2, 2, 64, 4, True)])
def test_gemm_umma_qkv_epilogue(ops, m, nh, nkv, k, ps, with_bias):
    """The tcgen05 product of the stacked q, k, v projection with bias, rotation and cache write in its
    epilogue, against the product in float64 followed by the plain formulas; tokens with slot -1 leave the
    cache alone; an odd number of heads leaves the last tile half empty."""
    hd, g = 128, torch.Generator().manual_seed(90 + m)
    width = (nh + 2 * nkv) * hd
    x = (torch.randn((m, k), generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn((width, k), generator=g) / math.sqrt(k)).to(torch.bfloat16)
    bias = torch.randn((width,), generator=g) * 0.5 if with_bias else None
    ang = torch.randn((m, hd // 2), generator=g) * 3.0
    cos, sin = torch.cos(ang), torch.sin(ang)
    pages = (m + ps - 1) // ps + 3
    perm = torch.randperm(pages * ps, generator=g)[:m].to(torch.int32)
    perm[5] = -1
    perm[m - 1] = -1
    pool = torch.full((pages, 1, 2, nkv, ps, hd), 7.0, dtype=torch.bfloat16)
    # plain: float64 product, bias, rotate-half
    prod = x.double() @ w.double().t()
    if bias is not None:
        prod = prod + bias.double()
    heads = prod.view(m, nh + 2 * nkv, hd)
    lo, hi = heads[:, :nh + nkv, :hd // 2], heads[:, :nh + nkv, hd // 2:]
    c, s_ = cos.double()[:, None, :], sin.double()[:, None, :]
    rot = torch.cat([lo * c - hi * s_, hi * c + lo * s_], dim=-1)
    want_q, want_k, want_v = rot[:, :nh], rot[:, nh:], heads[:, nh + nkv:]
    xd, wd, pd = x.to(DEV), w.to(DEV), pool.to(DEV)
    q_out = torch.full((m, width), 3.0, dtype=torch.bfloat16, device=DEV)
    ops.gemm_umma_qkv(xd, wd, None if bias is None else bias.to(DEV), q_out, cos.to(DEV), sin.to(DEV), perm.to(DEV),
                      pd[0, 0, 0], pd[0, 0, 1], pd.stride(0), ps, nh, nkv)
    ops.check_device_errors(DEV)
    _close(q_out[:, :nh * hd].float().cpu(), want_q.reshape(m, nh * hd).float(), 6e-3, "rotated queries")
    assert torch.all(q_out[:, nh * hd:] == 3.0), "columns beyond the queries were written"
    got = pd.float().cpu()
    seen = torch.zeros((pages, ps), dtype=torch.bool)
    for t in range(m):
        sl = int(perm[t])
        if sl < 0:
            continue
        seen[sl // ps, sl % ps] = True
        _close(got[sl // ps, 0, 0, :, sl % ps], want_k[t].float(), 6e-3, f"key of token {t}")
        _close(got[sl // ps, 0, 1, :, sl % ps], want_v[t].float(), 6e-3, f"value of token {t}")
    untouched = got.permute(0, 4, 1, 2, 3, 5)[~seen]
    assert torch.all(untouched == 7.0), "a slot that belongs to no token was written"
    # beside the library product followed by the kernel that does the same on its bfloat16 rows
    qkv = ops.matmul_library(xd, wd, torch.bfloat16)
    pd2 = pool.to(DEV)
    ops.qkv_rope_kv_write(qkv, None if bias is None else bias.to(DEV), cos.to(DEV), sin.to(DEV), perm.clamp(min=0).to(DEV),
                          pd2[0, 0, 0], pd2[0, 0, 1], pd2.stride(0), ps, nh, nkv, hd)
    _close(q_out[:, :nh * hd].float().cpu(), qkv[:, :nh * hd].float().cpu(), 3e-2, "beside the separate kernels")


def test_gemm_umma_qkv_epilogue_queries_only(ops):
    """A layer that reads another layer's cache has only queries: no slot map, no cache."""
    m, nh, k, hd, g = 260, 3, 136, 128, torch.Generator().manual_seed(95)
    x = (torch.randn((m, k), generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn((nh * hd, k), generator=g) / math.sqrt(k)).to(torch.bfloat16)
    bias = torch.randn((nh * hd,), generator=g) * 0.5
    ang = torch.randn((m, hd // 2), generator=g) * 3.0
    cos, sin = torch.cos(ang), torch.sin(ang)
    heads = (x.double() @ w.double().t() + bias.double()).view(m, nh, hd)
    lo, hi, c, s_ = heads[..., :hd // 2], heads[..., hd // 2:], cos.double()[:, None, :], sin.double()[:, None, :]
    want = torch.cat([lo * c - hi * s_, hi * c + lo * s_], dim=-1).reshape(m, nh * hd)
    q_out = torch.empty((m, nh * hd), dtype=torch.bfloat16, device=DEV)
    ops.gemm_umma_qkv(x.to(DEV), w.to(DEV), bias.to(DEV), q_out, cos.to(DEV), sin.to(DEV), None, None, None, 0, 16, nh, 0)
    ops.check_device_errors(DEV)
    _close(q_out.float().cpu(), want.float(), 6e-3, "rotated queries")


# --------------------------------------------------------------------- sampling
def test_qkv_rope_from_partial_sums(ops):
    """The RoPE + cache-write kernel given float32 partial sums of the product
    gives what it gives for their sum rounded to bfloat16 up to that rounding,
    and exactly what it gives when the sum is exact in bfloat16."""
    nh, nkv, hd, ps, n = 5, 2, 32, 8, 7
    width = (nh + 2 * nkv) * hd
    parts = (torch.randint(-8, 9, (3, n, width), generator=torch.Generator().manual_seed(60)).float() / 4).to(DEV)
    total = parts.sum(0)                                  # multiples of 1/4 below 8: exact in bfloat16
    bias = _rand((width,), torch.float32, 61)
    ang = _rand((n, hd // 2), torch.float32, 62)
    cos, sin = torch.cos(ang), torch.sin(ang)
    slots = torch.tensor([3, 17, 9, 0, 30, 31, 12], dtype=torch.int32, device=DEV)
    def run(partials):
        pool = torch.zeros((4, 1, 2, nkv, ps, hd), dtype=torch.bfloat16, device=DEV)
        qkv = torch.zeros((n, width), dtype=torch.bfloat16, device=DEV) if partials is not None else total.to(torch.bfloat16)
        ops.qkv_rope_kv_write(qkv, bias, cos, sin, slots, pool[0, 0, 0], pool[0, 0, 1], pool.stride(0), ps, nh, nkv, hd, partials)
        return qkv[:, :nh * hd].clone(), pool
    q1, pool1 = run(None)
    q2, pool2 = run(parts)
    assert torch.equal(q1, q2) and torch.equal(pool1, pool2)


def test_argmax_lowest_index_among_equal_maxima(ops):
    v = 152064
    logits = _rand((5, v), torch.float32, 30)
    logits[0, 77] = logits[0, 150000] = 50.0
    logits[1, v - 1] = 60.0
    logits[2, 0] = 60.0
    logits[3, :] = 1.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.argmax(logits, out)
    want = [77, v - 1, 0, 0, int(torch.argmax(logits[4].cpu()))]
    assert out.tolist() == want
    assert host.argmax(logits.cpu(), torch.empty(5, dtype=torch.int32)).tolist() == want
    # a strided view (rows of a wider buffer)
    wide = torch.zeros((3, 1000), device=DEV)
    wide[:, 300] = 1.0
    out2 = torch.empty(3, dtype=torch.int32, device=DEV)
    ops.argmax(wide[:, :777], out2)
    assert out2.tolist() == [300, 300, 300]


@pytest.mark.parametrize("v", [4096, 10007, 33333, 152064])
def test_argmax_of_wide_rows_in_slices(ops, v):
    """Wide rows are cut into slices (one block each): maxima on the borders of
    slices, equal maxima in different slices, NaNs, rows that are not 16-byte
    aligned (an odd row stride)."""
    parts = min(64, v // 2048)
    slice_len = ((v + parts - 1) // parts + 3) // 4 * 4
    for stride in (v, v + 1):
        buf = _rand((6, stride), torch.float32, 32 + v % 7)
        logits = buf[:, :v]
        logits[0, slice_len - 1] = 70.0                      # last element of the first slice
        logits[1, slice_len] = 70.0                          # first element of the second
        logits[2, v - 1] = logits[2, slice_len + 5] = 70.0   # equal maxima in two slices: the lower index
        logits[3, :] = float("nan")
        logits[3, v - 3] = -5.0                              # the only number of the row
        logits[4, 17] = float("nan")
        logits[4, v // 2] = 80.0
        out = torch.empty(6, dtype=torch.int32, device=DEV)
        ops.argmax(logits, out)
        assert out.tolist() == [slice_len - 1, slice_len, slice_len + 5, v - 3, v // 2,
                                int(torch.argmax(logits[5].cpu()))], (v, stride)
        assert host.argmax(logits.cpu(), torch.empty(6, dtype=torch.int32)).tolist() == out.tolist()


def test_penalties(ops):
    v = 1000
    logits = _rand((3, v), torch.float32, 31)
    want = logits.clone().cpu()
    ids = torch.tensor([[5, 9, 700, 0], [1, 2, 3, 4], [0, 0, 0, 0]], dtype=torch.int32)
    cnt = torch.tensor([[2, 1, 5, 0], [1, 1, 1, 1], [0, 0, 0, 0]], dtype=torch.int32)
    n = torch.tensor([3, 4, 0], dtype=torch.int32)
    rep, freq, pres = torch.tensor([1.3, 1.0, 2.0]), torch.tensor([0.1, 0.5, 0.0]), torch.tensor([0.2, 0.0, 0.0])
    ref.apply_penalties(want, ids, cnt, n, rep, freq, pres)
    ops.apply_penalties(logits, ids.to(DEV), cnt.to(DEV), n.to(DEV), rep.to(DEV), freq.to(DEV), pres.to(DEV))
    _close(logits, want, 1e-6, "penalties")


def test_penalties_from_rings_on_the_device(ops):
    """The penalties counted from each request's ring of tokens on the device are those counted on the host
    from the same tokens: windows shorter and longer than what the request has, rings that have wrapped
    around, rows without penalties, tokens appended by the kernel."""
    v, size, n_slots = 700, 16, 6
    g = torch.Generator().manual_seed(44)
    history = [torch.randint(0, 40, (n,), generator=g).tolist() for n in (5, 16, 23, 40, 0, 9)]   # per slot, 0..39: many repeats
    ring = torch.zeros((n_slots, size), dtype=torch.int32, device=DEV)
    totals = torch.zeros(n_slots, dtype=torch.int32, device=DEV)
    one = lambda x: torch.tensor([x], dtype=torch.int32, device=DEV)
    for slot, h in enumerate(history):                       # token by token, through the append kernel
        for t in h:
            ops.ring_append(ring, totals, one(slot), one(t))
    assert totals.tolist() == [len(h) for h in history]
    rows = [(3, 8, 1.3, 0.2, 0.5), (1, 16, 1.0, 0.7, 0.0), (0, 64, 2.0, 0.0, 0.0), (-1, 8, 1.5, 0.5, 0.5),
            (2, 5, 1.1, 0.1, 0.1), (4, 8, 1.7, 0.3, 0.2), (5, 1, 1.2, 0.0, 1.0)]      # slot, window, rep, freq, pres
    logits = _rand((len(rows), v), torch.float32, 45, 2.0)
    want = logits.clone().cpu()
    for i, (slot, window, rep, freq, pres) in enumerate(rows):
        if slot < 0:
            continue
        n = min(window, size, len(history[slot]))
        seen = history[slot][len(history[slot]) - n:]
        ids = sorted(set(seen))
        ref.apply_penalties(want[i:i + 1], torch.tensor([ids]), torch.tensor([[seen.count(t) for t in ids]]),
                            torch.tensor([len(ids)]), torch.tensor([rep]), torch.tensor([freq]), torch.tensor([pres]))
    f = lambda vals, dt: torch.tensor(vals, dtype=dt, device=DEV)
    ops.apply_penalties_ring(logits, ring, totals, f([r[0] for r in rows], torch.int32), f([r[1] for r in rows], torch.int32),
                             f([r[2] for r in rows], torch.float32), f([r[3] for r in rows], torch.float32),
                             f([r[4] for r in rows], torch.float32))
    _close(logits, want, 1e-6, "penalties from the rings")


def _sample(ops, logits, temperature, top_k, top_p, min_p, seeds, counters):
    r, v = logits.shape
    f = lambda x, dt: torch.tensor(x, dtype=dt, device=DEV)
    out = torch.empty(r, dtype=torch.int32, device=DEV)
    ops.sample(logits, torch.empty(r * v, dtype=torch.float32, device=DEV), f(temperature, torch.float32),
               f(top_k, torch.int32), f(top_p, torch.float32), f(min_p, torch.float32), f(seeds, torch.int64),
               f(counters, torch.int64), out)
    return out.tolist()


@pytest.mark.parametrize("v,r,offset", [(1000, 64, 0), (152064, 16, 0), (40000, 8, 1), (8193, 8, 3), (420000, 4, 0)])
def test_sample_matches_inverse_cdf(ops, v, r, offset):
    """For each row the drawn token is the one whose cumulative-probability
    interval (over the kept tokens, in index order) contains the row's uniform.
    Rows short enough for one block, rows spread over a cluster of 2 to 8
    blocks, rows that start off a 16-byte boundary, and rows too long for a
    cluster's shared memory (the kernel that keeps its weights in scratch)."""
    import plain_qwen2 as plain
    wide = _rand((r, v + offset), torch.float32, 32, 3.0)
    logits = wide[:, offset:]
    temps = [0.8 if i % 2 else 1.3 for i in range(r)]
    ks = [0, 5, 50, 0][0:4] * (r // 4)
    ps = [1.0, 1.0, 0.9, 0.5] * (r // 4)
    mps = [0.0, 0.0, 0.0, 0.05] * (r // 4)
    seeds, counters = [1234 + i for i in range(r)], [i * 7 for i in range(r)]
    got = _sample(ops, logits, temps, ks, ps, mps, seeds, counters)
    for i in range(r):
        kept = plain.kept_probabilities(logits[i].cpu(), temps[i], ks[i], ps[i], mps[i])
        assert kept[got[i]] > 0, f"row {i}: token {got[i]} is outside the kept set"
        cdf = torch.cumsum(kept, 0) / kept.sum()
        u = ref.uniform01(seeds[i], counters[i])
        lo = float(cdf[got[i] - 1]) if got[i] > 0 else 0.0
        assert lo - 1e-5 <= u <= float(cdf[got[i]]) + 1e-5, f"row {i}: u={u} not in [{lo}, {float(cdf[got[i]])}]"
        # the C++ loops: the same kept set, and the same token unless u lies within rounding of an interval's end
        kept_c = host.kept_probabilities(logits[i].cpu().contiguous(), temps[i], ks[i], ps[i], mps[i])
        assert torch.equal(kept_c > 0, kept > 0) and float((kept_c - kept).abs().max()) < 1e-7   # float32 temperature there
        assert host.uniform01(seeds[i], counters[i]) == u
        tok_c = host.inverse_cdf(kept_c, u)
        assert tok_c == got[i] or min(abs(u - lo), abs(u - float(cdf[got[i]]))) < 1e-5, (i, tok_c, got[i])


def test_sample_thresholds_at_ties_and_edges(ops):
    """top-k keeps every token that ties with the k-th; top-p 'the smallest set of the largest that reaches p'
    with ties at the cut kept; a row of equal logits; one finite logit among -inf; NaN never drawn."""
    v = 20000
    base = torch.full((6, v), -30.0)                      # weights that add up to nothing beside the few set below
    base[0, [7, 900, 19999]] = 2.0                       # three equal maxima, top-k 2: all three stay, nothing else
    base[1, 11], base[1, 12], base[1, 13] = 3.0, 2.0, 2.0   # top-p 0.6: the maximum alone has < 0.6 -> both ties join
    base[2] = 0.25                                        # all equal: any token, uniform over the row
    base[3] = float("-inf"); base[3, 4242] = -1.0        # one finite logit
    base[4, 5] = float("nan"); base[4, 6] = 1.0           # NaN never wins nor is drawn
    base[5, 100:200] = 1.0                                # top-k 10 with 100 equal maxima: all 100 stay
    logits = base.to(DEV)
    n = 200
    seen = [set() for _ in range(6)]
    for c in range(n):
        got = _sample(ops, logits, [1.0] * 6, [2, 0, 0, 0, 1, 10], [1.0, 0.6, 1.0, 1.0, 1.0, 1.0], [0.0] * 6,
                      [5, 6, 7, 8, 9, 10], [c] * 6)
        for i in range(6):
            seen[i].add(got[i])
    assert seen[0] == {7, 900, 19999}
    assert seen[1] == {11, 12, 13}
    assert len(seen[2]) > 150 and min(seen[2]) < 2000 and max(seen[2]) > 18000
    assert seen[3] == {4242}
    assert seen[4] == {6}
    assert seen[5] <= set(range(100, 200)) and len(seen[5]) > 60


def test_sample_distribution_and_determinism(ops):
    v, draws = 50, 4000
    base = _rand((1, v), torch.float32, 33, 1.5)
    logits = base.expand(draws, v).contiguous()
    got = _sample(ops, logits, [1.0] * draws, [0] * draws, [1.0] * draws, [0.0] * draws, [99] * draws,
                  list(range(draws)))
    again = _sample(ops, logits, [1.0] * draws, [0] * draws, [1.0] * draws, [0.0] * draws, [99] * draws,
                    list(range(draws)))
    assert got == again
    p = torch.softmax(base[0].double().cpu(), 0)
    counts = torch.bincount(torch.tensor(got), minlength=v).double()
    chi2 = float(((counts - draws * p) ** 2 / (draws * p)).sum())
    assert chi2 < 110.0, f"chi-square {chi2:.1f} over {v - 1} degrees of freedom"   # p ~ 1e-6 under the null
    # temperature 0 = argmax; rows are independent of their neighbours
    mixed = _sample(ops, logits[:4], [0.0, 1.0, 0.0, 1.0], [0] * 4, [1.0] * 4, [0.0] * 4, [99] * 4, [0, 1, 2, 3])
    am = int(torch.argmax(base[0].cpu()))
    assert mixed[0] == am and mixed[2] == am and mixed[1] == got[1] and mixed[3] == got[3]


@pytest.mark.parametrize("odt", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (300, 520, 200), (2048, 4608, 3584), (17, 40, 72), (513, 1000, 1096),
                                   (1024, 3584, 512), (2048, 3584, 256)])
def test_gemm_umma(ops, m, n, k, odt):
    """The tcgen05 product against float64, with tiles cut by M, N and K (TMA fills
    the missing rows and the K tail with zeros), with and without bias."""
    x, w, b = _rand((m, k), torch.bfloat16, 50), _rand((n, k), torch.bfloat16, 51, 0.1), _rand((n,), torch.float32, 52)
    want = x.double().cpu() @ w.double().cpu().T
    for bias in (None, b):
        out = torch.full((m, n), float("nan"), dtype=odt, device=DEV)
        ops.gemm_umma(x, w, bias, out)
        ops.check_device_errors(DEV)
        _close(out, want + (0 if bias is None else b.double().cpu()), 1e-5 if odt == torch.float32 else 6e-3, "gemm_umma")
    # rows of a wider buffer as input (a row stride that is not K)
    wide = _rand((m, k + 24), torch.bfloat16, 53)
    out = torch.empty((m, n), dtype=odt, device=DEV)
    ops.gemm_umma(wide[:, 8:8 + k], w, None, out)
    _close(out, wide[:, 8:8 + k].double().cpu() @ w.double().cpu().T, 1e-5 if odt == torch.float32 else 6e-3, "strided rows")


def test_gemm_umma_one_hot(ops):
    """Each output picks one product: a wrong row, column or K slice of a tile shows as a wrong value."""
    m, n, k = 512, 768, 256
    x = torch.zeros((m, k), dtype=torch.bfloat16, device=DEV)
    w = torch.zeros((n, k), dtype=torch.bfloat16, device=DEV)
    rows = torch.arange(m, device=DEV)
    x[rows, rows % k] = (1 + rows % 7).to(torch.bfloat16)
    cols = torch.arange(n, device=DEV)
    w[cols, (cols * 5) % k] = (1 + cols % 5).to(torch.bfloat16)
    out = torch.empty((m, n), dtype=torch.float32, device=DEV)
    ops.gemm_umma(x, w, None, out)
    ops.check_device_errors(DEV)
    assert torch.equal(out, x.float() @ w.float().T)


@pytest.mark.parametrize("m,inter,k", [(256, 128, 64), (700, 1000, 328), (2048, 18944, 3584)])
def test_gemm_umma_swiglu(ops, m, inter, k):
    x, w = _rand((m, k), torch.bfloat16, 54), _rand((2 * inter, k), torch.bfloat16, 55, 0.2)
    out = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_umma(x, w, None, out, swiglu=True)
    ops.check_device_errors(DEV)
    gu = x.double().cpu() @ w.double().cpu().T
    gate, up = gu[:, :inter], gu[:, inter:]
    _close(out, gate / (1 + torch.exp(-gate)) * up, 6e-3, "gemm_umma swiglu")


@pytest.mark.parametrize("m", [1, 17, 32, 40, 64, 100, 256])
@pytest.mark.parametrize("n,k", [(3584, 3584), (4608, 3584), (3584, 18944), (100, 96), (300, 1096), (257, 64)])
def test_gemm_umma_skinny(ops, m, n, k):
    """The tcgen05 product for a few rows (weights as the tiles' rows, K cut into parts that the consumer adds)
    against float64: rows and columns that do not fill a tile, K with a tail, one-hot rows that tell the
    transposed store apart from a plain one."""
    x, w = _rand((m, k), torch.bfloat16, 80), _rand((n, k), torch.bfloat16, 81, 0.1)
    x[m // 2] = 0
    x[m // 2, k // 3] = 1.0                                # this row of the result is column k // 3 of w
    parts = ops.gemm_umma_skinny_parts(n, k)
    out = torch.full((parts, m, n), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_umma_skinny(x, w, out)
    ops.check_device_errors(DEV)
    got = out.double().sum(0).cpu()
    want = x.double().cpu() @ w.double().cpu().T
    assert torch.isfinite(out).all()
    _close(got, want, 1e-5, f"few-row product in {parts} parts")
    assert torch.equal(got[m // 2].float(), w[:, k // 3].float().cpu())


def test_gemv_plan_depends_on_the_matrix_only(ops):
    """The number of K parts is the kernel's own choice from the matrix sizes; it
    is within bounds, repeatable, and 1 where K is too short to cut."""
    for n, k in ((3584, 3584), (4608, 3584), (3584, 18944), (48, 64), (1000, 520)):
        s = ops.gemv_k_splits(n, k)
        assert 1 <= s <= 8 and s == ops.gemv_k_splits(n, k)
        assert s == 1 or (k + 31) // 32 // s >= 16
    assert ops.gemv_k_splits(48, 64) == 1
