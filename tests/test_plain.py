"""The plain implementation checked against itself: properties that hold for
the formulas whatever the weights are (no GPU)."""
from __future__ import annotations

import math

import torch

import plain_qwen2 as plain
from helpers import TINY_A, TINY_B, TINY_E, make_model_folder, random_tokens


def test_rms_norm():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = plain.rms_norm(x, torch.tensor([2.0, 0.5], dtype=torch.float64), 0.0)
    rms = math.sqrt((9 + 16) / 2)
    assert torch.allclose(y, torch.tensor([[3 / rms * 2, 4 / rms * 0.5]], dtype=torch.float64))


def test_rope_is_a_rotation_by_relative_position():
    d = 16
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, d, generator=g, dtype=torch.float64), torch.randn(1, 1, d, generator=g, dtype=torch.float64)

    def dot(pq, pk):
        cq, sq = plain.rope_angles(torch.tensor([pq]), d, 10000.0, torch.float64)
        ck, sk = plain.rope_angles(torch.tensor([pk]), d, 10000.0, torch.float64)
        return float((plain.apply_rope_half(q, cq, sq) * plain.apply_rope_half(k, ck, sk)).sum())
    assert abs(dot(5, 3) - dot(105, 103)) < 1e-9          # depends on the distance only
    c0, s0 = plain.rope_angles(torch.tensor([0]), d, 10000.0, torch.float64)
    assert torch.equal(plain.apply_rope_half(q, c0, s0), q)  # position 0 leaves the vector alone
    c, s = plain.rope_angles(torch.tensor([9]), d, 10000.0, torch.float64)
    r = plain.apply_rope_half(q, c, s)
    assert abs(float(r.norm() - q.norm())) < 1e-12
    # pairs are (i, i + d/2): rotating by hand
    a = 9 * 10000.0 ** (-2 * 3 / d)
    assert abs(float(r[0, 0, 3]) - (float(q[0, 0, 3]) * math.cos(a) - float(q[0, 0, 11]) * math.sin(a))) < 1e-12


def test_attention_is_causal_and_windowed():
    g = torch.Generator().manual_seed(1)
    t, nh, nkv, d = 12, 4, 2, 8
    q, k, v = (torch.randn(t, n, d, generator=g, dtype=torch.float64) for n in (nh, nkv, nkv))
    full = plain.causal_gqa_attention(q, k, v, 0.3)
    k2, v2 = k.clone(), v.clone()
    k2[7:], v2[7:] = 99.0, -99.0                            # the future does not matter
    assert torch.equal(plain.causal_gqa_attention(q, k2, v2, 0.3)[:7], full[:7])
    assert torch.allclose(full[0], v[0].repeat_interleave(nh // nkv, 0))   # the first token sees itself only
    win = plain.causal_gqa_attention(q, k, v, 0.3, window=3)
    k3, v3 = k.clone(), v.clone()
    k3[:6], v3[:6] = 50.0, 50.0                              # token 8 with window 3 sees 6, 7, 8
    assert torch.allclose(plain.causal_gqa_attention(q, k3, v3, 0.3, window=3)[8], win[8])
    assert not torch.allclose(plain.causal_gqa_attention(q, k3, v3, 0.3, window=4)[8], win[8])
    assert torch.allclose(plain.causal_gqa_attention(q, k, v, 0.3, window=100), full)


def test_forward_prefix_property_and_tied_head(tmp_path):
    for name, cfg in (("a", TINY_A), ("b", TINY_B), ("e", TINY_E)):
        folder = make_model_folder(cfg, 2, str(tmp_path / name))
        c, w = plain.load_folder(folder)
        toks = random_tokens(cfg["vocab_size"], 60, 9)
        full = plain.forward(c, w, toks)
        assert full.shape == (60, cfg["vocab_size"]) and bool(torch.isfinite(full).all())
        assert torch.allclose(plain.forward(c, w, toks[:25]), full[:25], atol=1e-12)   # causal: a prefix is enough
        assert ("lm_head.weight" in w) == (not cfg["tie_word_embeddings"])
    # float32 arithmetic agrees with float64 to float32 accuracy
    c32, w32 = plain.load_folder(folder, torch.float32)
    assert float((plain.forward(c32, w32, toks).double() - full).abs().max()) < 1e-4 * float(full.abs().max())


def test_kept_probabilities():
    logits = torch.log(torch.tensor([0.5, 0.25, 0.125, 0.0625, 0.0625]))
    p = plain.kept_probabilities(logits, 1.0, 0, 1.0, 0.0)
    assert torch.allclose(p, torch.tensor([0.5, 0.25, 0.125, 0.0625, 0.0625], dtype=torch.float64))
    assert (plain.kept_probabilities(logits, 1.0, 2, 1.0, 0.0) > 0).tolist() == [True, True, False, False, False]
    assert (plain.kept_probabilities(logits, 1.0, 0, 0.7, 0.0) > 0).tolist() == [True, True, False, False, False]
    assert (plain.kept_probabilities(logits, 1.0, 0, 0.76, 0.0) > 0).tolist() == [True, True, True, False, False]
    assert (plain.kept_probabilities(logits, 1.0, 0, 1.0, 0.2) > 0).tolist() == [True, True, True, False, False]
