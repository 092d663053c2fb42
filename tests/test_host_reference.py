"""The host-side C++ reference (csrc/host_reference) against the plain
implementation: every operation alone, and the whole model stepped over its own
paged cache in portions, single tokens and mixed batches, with scattered pages.
Both rest on the same formulas of the reference but share no code: one is
PyTorch in float64 on whole sequences, the other C++ loops in float32 over a
paged cache.  Needs no GPU."""
from __future__ import annotations

import math
import random

import pytest
import torch

import kernel_refs
import plain_qwen2 as plain
from helpers import TINY, make_model_folder, random_tokens
from inferflux_b200.kernels import host_reference as host


def _rand(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


def _close(got, want, tol, what):
    err = float((got.double() - want.double()).abs().max() / want.double().abs().max())
    assert err <= tol, f"{what}: {err:.3e}"


def test_norm_swiglu_gemm_embedding():
    x, w = _rand((5, 100), 1), _rand((100,), 2) + 1.0
    delta = _rand((3, 5, 100), 3)
    res = x.clone()
    out = torch.empty((5, 100))
    host.add_rmsnorm(res, delta, w, 1e-5, out, n_partials=3)
    summed = x.double() + delta.double().sum(0)
    _close(res, summed, 1e-6, "residual")
    _close(out, plain.rms_norm(summed, w.double(), 1e-5), 1e-6, "norm")
    rows = torch.tensor([4, 0, 4], dtype=torch.int32)
    out2 = torch.empty((3, 100))
    before = res.clone()
    host.add_rmsnorm(res, None, w, 1e-5, out2, rows)
    assert torch.equal(res, before) and torch.equal(out2[0], out2[2])
    _close(out2, plain.rms_norm(summed, w.double(), 1e-5)[[4, 0, 4]], 1e-6, "gathered rows")
    gu = _rand((4, 2 * 37), 4, 2.0)
    act = host.swiglu(gu, torch.empty((4, 37)))
    _close(act, plain.silu_mul(gu[:, :37].double(), gu[:, 37:].double()), 1e-6, "swiglu")
    a, m, b = _rand((7, 257), 5), _rand((33, 257), 6), _rand((33,), 7)
    _close(host.gemm(a, m, b, torch.empty((7, 33))), a.double() @ m.double().T + b.double(), 1e-6, "gemm")
    table = _rand((50, 24), 8)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
    assert torch.equal(host.embed_gather(table, ids, torch.empty((4, 24))), plain.embed(table, ids.tolist()))


@pytest.mark.parametrize("nh,nkv,hd,rot,ps", [(4, 2, 16, 16, 16), (3, 1, 32, 32, 4), (10, 2, 48, 24, 8)])
def test_rotation_and_cache_write(nh, nkv, hd, rot, ps):
    n, pages = 11, 6
    positions = torch.tensor([0, 1, 2, 500, 501, 4095, 31, 32, 33, 7, 8], dtype=torch.int32)
    inv = torch.pow(torch.tensor(1e6, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)
    cos, sin = torch.empty((n, rot // 2)), torch.empty((n, rot // 2))
    host.rope_table(positions, inv, cos, sin)
    c64, s64 = plain.rope_angles(positions, rot, 1e6, torch.float64)
    _close(cos, c64, 1e-6, "cos"), _close(sin, s64, 1e-6, "sin")
    width = (nh + 2 * nkv) * hd
    qkv, bias = _rand((n, width), 9), _rand((width,), 10)
    pool = torch.zeros((pages, 2, 2, nkv, ps, hd))
    slots = torch.randperm(pages * ps, generator=torch.Generator().manual_seed(1))[:n].int()
    slots[2] = -1
    x = (qkv.double() + bias.double()).view(n, nh + 2 * nkv, hd)
    want = plain.apply_rope_half(x[:, :nh + nkv], c64, s64)
    host.qkv_rope_kv_write(qkv, bias, cos, sin, slots, pool[0, 1, 0], pool[0, 1, 1], pool.stride(0), ps, nh, nkv, hd)
    _close(qkv[:, :nh * hd].reshape(n, nh, hd), want[:, :nh], 2e-6, "rotated q")
    for t in range(n):
        s = int(slots[t])
        if s < 0:
            continue
        _close(pool[s // ps, 1, 0, :, s % ps], want[t, nh:], 2e-6, "cached k")
        _close(pool[s // ps, 1, 1, :, s % ps], x[t, nh + nkv:], 2e-6, "cached v")
    assert float(pool[:, 0].abs().max()) == 0.0 and float(pool.abs().sum()) > 0


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, None), (3, 1, 32, 24), (10, 2, 48, None), (7, 1, 128, 100)])
def test_attention_over_pages(nh, nkv, hd, window):
    """Queries of a later portion over keys that lie in scattered pages equal the
    plain attention over the whole sequence."""
    ps, total, new = 8, 150, 41
    g = torch.Generator().manual_seed(hd)
    q, k, v = (torch.randn((total, h, hd), generator=g) for h in (nh, nkv, nkv))
    k[5] *= 3.0
    q[-1] = k[5].repeat_interleave(nh // nkv, dim=0)             # the last query looks far back (or just out of its window)
    blocks = (total + ps - 1) // ps
    perm = torch.randperm(blocks + 4, generator=g).tolist()[:blocks]
    pool = torch.zeros((blocks + 4, 1, 2, nkv, ps, hd))
    for pos in range(total):
        pool[perm[pos // ps], 0, 0, :, pos % ps] = k[pos]
        pool[perm[pos // ps], 0, 1, :, pos % ps] = v[pos]
    it = lambda x: torch.tensor(x, dtype=torch.int32)
    out = torch.zeros((new, nh * hd))
    qn = q[total - new:].reshape(new, nh * hd).contiguous()
    host.attention_paged(qn, nh * hd, out, pool[0, 0, 0], pool[0, 0, 1], pool.stride(0), ps, it([perm]), it([0]),
                         it([new]), it([total - new]), nh, nkv, hd, 1 / math.sqrt(hd), window)
    want = plain.causal_gqa_attention(q.double(), k.double(), v.double(), 1 / math.sqrt(hd), window)[total - new:]
    _close(out.view(new, nh, hd), want, 2e-6, "paged attention")


def test_sampling_pieces():
    v = 300
    logits = _rand((v,), 11, 3.0)
    logits[7] = logits[9] = float(logits.max()) + 1.0            # two equal maxima
    for t, k, p, mp in [(1.0, 0, 1.0, 0.0), (0.7, 5, 1.0, 0.0), (1.3, 0, 0.6, 0.0), (1.0, 0, 1.0, 0.05),
                        (0.9, 40, 0.8, 0.01), (1.0, 1, 1.0, 0.0)]:
        want = plain.kept_probabilities(logits, t, k, p, mp)
        got = host.kept_probabilities(logits, t, k, p, mp)
        assert torch.equal(got > 0, want > 0), (t, k, p, mp)
        assert float((got - want).abs().max()) < 1e-7            # the C++ side takes the temperature as a float32
    probs = torch.tensor([0.0, 0.5, 0.0, 0.25, 0.25], dtype=torch.float64)
    assert [host.inverse_cdf(probs, u) for u in (0.0, 0.49, 0.5, 0.74, 0.75, 0.999)] == [1, 1, 3, 3, 4, 4]
    assert host.uniform01(1234, 77) == kernel_refs.uniform01(1234, 77)
    assert host.argmax(torch.tensor([[1.0, 5.0, 5.0], [float("nan"), -2.0, -3.0]]),
                       torch.empty(2, dtype=torch.int32)).tolist() == [1, 1]
    lg = _rand((2, 50), 12)
    want = lg.clone()
    ids, cnt = torch.tensor([[3, 9, 0], [1, 2, 4]], dtype=torch.int32), torch.tensor([[2, 1, 0], [1, 1, 3]], dtype=torch.int32)
    n, rep, freq, pres = torch.tensor([2, 3], dtype=torch.int32), torch.tensor([1.3, 2.0]), torch.tensor([0.1, 0.0]), torch.tensor([0.2, 0.5])
    host.apply_penalties(lg, ids, cnt, n, rep, freq, pres)
    for r in range(2):
        recent = [int(ids[r, k]) for k in range(int(n[r])) for _ in range(int(cnt[r, k]))]
        want[r] = plain.apply_penalties(want[r], recent, float(rep[r]), float(freq[r]), float(pres[r]))
    _close(lg, want, 1e-6, "penalties")


def _host_model(cfg, weights, num_pages, page_size):
    w32 = {k: v.float() for k, v in weights.items()}
    nh = cfg["num_attention_heads"]
    layers = cfg["num_hidden_layers"]
    return host.HostModel(cfg["hidden_size"], nh, cfg.get("num_key_value_heads", nh),
                          cfg.get("head_dim") or cfg["hidden_size"] // nh, cfg["intermediate_size"], cfg["vocab_size"],
                          layers, cfg.get("rms_norm_eps", 1e-6), cfg.get("rope_theta", 10000.0),
                          bool(cfg.get("tie_word_embeddings")), w32, [plain.window_of_layer(cfg, i) for i in range(layers)],
                          num_pages, page_size)


@pytest.mark.parametrize("name", ["A", "B", "E"])
def test_whole_model_in_portions_and_mixed_batches(tmp_path, name):
    """Three requests stepped through the C++ model over one shared pool of
    scattered pages: portions of changing size beside single tokens of the
    others; every position's logits equal the plain implementation's."""
    cfg = TINY[name]
    folder = make_model_folder(cfg, 3, str(tmp_path / "m"), sharpen=4.0)
    c, w = plain.load_folder(folder)
    ps = 4
    seqs = [random_tokens(cfg["vocab_size"], n, 20 + n) for n in (45, 23, 9)]
    refs = [plain.forward(c, w, s) for s in seqs]
    model = _host_model(c, w, 40, ps)
    rng = random.Random(5)
    free = list(range(40))
    rng.shuffle(free)
    tables, done = [[] for _ in seqs], [0] * len(seqs)
    worst = 0.0
    while any(d < len(s) for d, s in zip(done, seqs)):
        entries, checks = [], []
        for i, s in enumerate(seqs):
            left = len(s) - done[i]
            if left == 0 or rng.random() < 0.2:
                continue
            n = min(left, rng.choice([1, 1, 2, 3, 7, 16]))
            while len(tables[i]) * ps < done[i] + n:
                tables[i].append(free.pop())
            entries.append((tables[i], done[i], s[done[i]:done[i] + n], list(range(n))))
            checks.append((i, done[i], n))
            done[i] += n
        if not entries:
            continue
        logits = model.step(entries)
        row = 0
        for i, start, n in checks:
            err = float((logits[row:row + n].double() - refs[i][start:start + n]).abs().max() / refs[i].abs().max())
            worst = max(worst, err)
            row += n
    assert worst <= 1e-5, f"{name}: {worst:.3e}"
