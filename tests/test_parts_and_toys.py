"""Each part alone against the plain implementation, and the generality of
the layer description: a toy mixer with per-request state of its own that is
defined here, registered, built into a model and stepped without any change to
the package; a layer that runs twice; a layer that reads another run's cache; a
routed feed-forward; a position encoding with weights; a block with four norms;
a mixer that caches one latent vector per token instead of keys and values."""
from __future__ import annotations

import math
from types import SimpleNamespace

import pytest
import torch

import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def _rel(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def _rand(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


def _load(part, tensors, dtype):
    """Give a part its tensors the way the loader would: matrices in the engine's type, vectors float32."""
    part.load({k: (v.to(dtype) if v.dim() > 1 else v.float()).to(DEV) for k, v in tensors.items()})


# ------------------------------------------------------------------ parts alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_alone(dtype):
    from inferflux_b200.parts import RMSNorm
    h = 100
    part = RMSNorm(dict(name="n", hidden=h, eps=3e-6), "l", dtype, DEV)
    assert [w.name for w in RMSNorm.weight_specs(part.params, "l")] == ["l.n.weight"]
    w = 1 + _rand((h,), 1, 0.1)
    _load(part, {"l.n.weight": w}, dtype)
    res, delta = _rand((9, h), 2).to(DEV), _rand((9, h), 3).to(dtype).to(DEV)
    want_res = res.cpu().double() + delta.cpu().double()
    out = part.forward(res, delta)
    assert out.dtype == dtype
    assert _rel(res, want_res) < 1e-6
    assert _rel(out, plain.rms_norm(want_res, w.double(), 3e-6)) < TOL[dtype]


def test_rotary_alone():
    from inferflux_b200.parts import RotaryHalf
    part = RotaryHalf(dict(rotary_dim=48, theta=50000.0), "", torch.float32, DEV)
    pos = torch.tensor([0, 1, 17, 300, 4095], dtype=torch.int32, device=DEV)
    cos, sin = part.prepare(SimpleNamespace(n_tokens=5, positions=pos, device=DEV))
    wc, ws = plain.rope_angles(pos.cpu(), 48, 50000.0, torch.float64)
    assert cos.shape == (5, 24) and _rel(cos, wc) < 1e-6 and _rel(sin, ws) < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [3, 40])           # the weight-streaming kernel and the library product
def test_swiglu_alone(dtype, rows):
    from inferflux_b200.parts import SwiGLU
    h, inter = 96, 136
    part = SwiGLU(dict(name="mlp", hidden=h, intermediate=inter), "l", dtype, DEV)
    w = {"l.mlp.gate_proj.weight": _rand((inter, h), 4, 0.2), "l.mlp.up_proj.weight": _rand((inter, h), 5, 0.2),
         "l.mlp.down_proj.weight": _rand((h, inter), 6, 0.2)}
    w = {k: v.to(dtype).float() for k, v in w.items()}          # what the engine will really hold
    _load(part, dict(w), dtype)
    x = _rand((rows, h), 7).to(dtype)
    out = part.forward(x.to(DEV), None)
    from inferflux_b200.parts.base import PartialSums
    if isinstance(out, PartialSums):
        out = out.tensor.sum(0)
    want = plain.mlp_block(x.double(), {k: v.double() for k, v in w.items()}, "l.mlp")
    assert _rel(out, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_alone(dtype):
    from inferflux_b200.parts import LinearHead, TokenEmbedding
    v, h = 77, 40
    table = _rand((v, h), 8).to(dtype).float()
    emb = TokenEmbedding(dict(name="emb", vocab=v, hidden=h), "", dtype, DEV)
    _load(emb, {"emb.weight": table}, dtype)
    ids = torch.tensor([0, 76, 5, 5], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids).cpu(), table[ids.cpu().long()])
    head = LinearHead(dict(name="head", vocab=v, hidden=h, tied_to="emb.weight"), "", dtype, DEV)
    assert LinearHead.weight_specs(head.params, "")[0].kind == "ignored"
    head.load({"emb.weight": table.to(dtype).to(DEV)})
    x = _rand((6, h), 9).to(dtype)
    logits = head.forward(x.to(DEV))
    assert logits.dtype == torch.float32 and _rel(logits, x.double() @ table.double().T) < TOL[dtype]


def _one_layer_spec(hidden, nh, nkv, hd, window=None, extra_layers=(), schedule=None):
    from inferflux_b200.config.spec import LayerSpec, ModelSpec, PartSpec, Run
    norm = lambda name: PartSpec("rmsnorm", dict(name=name, hidden=hidden, eps=1e-6))
    attn = LayerSpec("layers.0", "prenorm", dict(
        mixer=PartSpec("gqa_attention", dict(name="attn", hidden=hidden, n_heads=nh, n_kv_heads=nkv, head_dim=hd,
                                             qkv_bias=True, o_bias=False, window=window)),
        mixer_norm=norm("n1"), feed_forward=PartSpec("swiglu", dict(name="mlp", hidden=hidden, intermediate=2 * hidden)),
        feed_forward_norm=norm("n2")), position="rope")
    layers = [attn, *extra_layers]
    return ModelSpec("Toy", hidden, 50, 512, PartSpec("token_embedding", dict(name="emb", vocab=50, hidden=hidden)),
                     norm("final"), PartSpec("linear_head", dict(name="head", vocab=50, hidden=hidden, tied_to=None)),
                     {"rope": PartSpec("rotary_half", dict(rotary_dim=hd, theta=10000.0))}, layers,
                     schedule or [Run(i) for i in range(len(layers))])


def _build(spec, dtype, seed, tokens=256, sharpen=4.0):
    from inferflux_b200.config import EngineConfig
    from inferflux_b200.engine import Model, StepRunner
    from inferflux_b200.weights.random_init import random_tensors
    model = Model(spec, dtype, DEV)
    tensors = random_tensors(model.weight_specs(), seed, torch.bfloat16, torch.float32, "cpu")
    for k in tensors:
        if k.endswith(("q_proj.weight", "k_proj.weight")):
            tensors[k] = (tensors[k].float() * sharpen).to(tensors[k].dtype)
    plain_w = {k: v.double() for k, v in tensors.items()}
    model.load({k: (v.to(dtype) if v.dim() > 1 else v.float()).to(DEV) for k, v in tensors.items()})
    runner = StepRunner(model, EngineConfig(dtype="float32" if dtype == torch.float32 else "bfloat16",
                                            kv_cache_tokens=tokens, max_seqs=4, cuda_graphs=False))
    return model, runner, plain_w


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, None), (6, 2, 64, 20)])
def test_attention_mixer_alone(dtype, nh, nkv, hd, window):
    """Only the mixer is called: normed input in, attention output out, first for a
    portion of 21 tokens, then for 12 more that attend over the cache."""
    from inferflux_b200.engine import StepEntry
    from inferflux_b200.parts.base import PartialSums
    hidden = 72
    model, runner, w = _build(_one_layer_spec(hidden, nh, nkv, hd, window), dtype, 11)
    mixer = model.blocks[0].mixer
    x = _rand((33, hidden), 12).to(dtype)
    want = plain.attention_block(x.double(), {k.replace("layers.0.attn", "a"): v for k, v in w.items()}, "a",
                                 torch.arange(33), nh, nkv, hd, 10000.0, window)
    outs = []
    for lo, hi in ((0, 21), (21, 33)):
        ctx = runner.build_context([StepEntry("r", [1] * (hi - lo), [])])
        ctx.position_tables["rope"] = model.positions["rope"].prepare(ctx)
        out = mixer.forward(x[lo:hi].to(DEV), ctx, model.runs[0], ctx.position_tables["rope"])
        outs.append(out.tensor.sum(0) if isinstance(out, PartialSums) else out.float())
        runner.kv.advance("r", hi - lo)
    assert _rel(torch.cat(outs), want) < TOL[dtype]


# ------------------------------------------------------- a toy mixer with state
def _register_running_mean():
    """out[t] = W * mean(x[0..t]): a mixer whose only memory is a running sum
    per request, kept in the request's state slot.  Defined in this test."""
    from inferflux_b200.config import register_part
    from inferflux_b200.parts.base import Part, StateNeed
    from inferflux_b200.weights.loader import MATRIX, WeightSpec

    class RunningMean(Part):
        family = "mixer"

        @classmethod
        def weight_specs(cls, params, prefix):
            h = int(params["hidden"])
            return [WeightSpec(cls.full_name(prefix, params, "mix.weight"), (h, h), MATRIX)]

        @classmethod
        def state_needs(cls, params):
            return [StateNeed("sum", (int(params["hidden"]),), torch.float32)]

        def load(self, tensors):
            self.w = tensors[self.full_name(self.prefix, self.params, "mix.weight")].float()

        def forward(self, x, ctx, run, position):
            out = torch.empty_like(x)
            state = run.states["sum"]
            for e, slot, start in zip(ctx.entries, ctx.slots, ctx.ctx_starts):
                q0 = ctx.entries.index(e)
                lo = sum(len(p.tokens) for p in ctx.entries[:q0])
                n = len(e.tokens)
                sums = state[slot] + torch.cumsum(x[lo:lo + n].float(), 0)
                counts = torch.arange(start + 1, start + n + 1, device=x.device, dtype=torch.float32)[:, None]
                out[lo:lo + n] = ((sums / counts) @ self.w.T).to(x.dtype)
                state[slot] = sums[-1]
            return out

    register_part("mixer", "running_mean", RunningMean)


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype):
    from inferflux_b200.config.spec import LayerSpec, PartSpec
    from inferflux_b200.engine import StepEntry
    _register_running_mean()
    hidden = 48
    norm = lambda name: PartSpec("rmsnorm", dict(name=name, hidden=hidden, eps=1e-6))
    toy = LayerSpec("layers.1", "prenorm", dict(
        mixer=PartSpec("running_mean", dict(name="rm", hidden=hidden)), mixer_norm=norm("n1"),
        feed_forward=PartSpec("swiglu", dict(name="mlp", hidden=hidden, intermediate=80)), feed_forward_norm=norm("n2")),
        position=None)
    spec = _one_layer_spec(hidden, 3, 1, 16, extra_layers=[toy])
    model, runner, w = _build(spec, dtype, 21)
    assert model.state_needs[1][0].name == "sum" and model.kv_needs[0].streams[0].heads == 1
    assert runner.state_storage.of_run(1)["sum"].shape == (4, hidden)

    def plain_forward(tokens):
        x = plain.embed(w["emb.weight"], tokens)
        h = plain.rms_norm(x, w["layers.0.n1.weight"], 1e-6)
        x = x + plain.attention_block(h, {k.replace("layers.0.attn", "a"): v for k, v in w.items()}, "a",
                                      torch.arange(len(tokens)), 3, 1, 16, 10000.0, None)
        x = x + plain.mlp_block(plain.rms_norm(x, w["layers.0.n2.weight"], 1e-6), w, "layers.0.mlp")
        h = plain.rms_norm(x, w["layers.1.n1.weight"], 1e-6)
        means = torch.cumsum(h, 0) / torch.arange(1, len(tokens) + 1, dtype=torch.float64)[:, None]
        x = x + means @ w["layers.1.rm.mix.weight"].T
        x = x + plain.mlp_block(plain.rms_norm(x, w["layers.1.n2.weight"], 1e-6), w, "layers.1.mlp")
        return plain.rms_norm(x, w["final.weight"], 1e-6) @ w["head.weight"].T

    toks_a = torch.randint(0, 50, (40,), generator=torch.Generator().manual_seed(1)).tolist()
    toks_b = torch.randint(0, 50, (23,), generator=torch.Generator().manual_seed(2)).tolist()
    want_a, want_b = plain_forward(toks_a), plain_forward(toks_b)
    # whole
    got = runner.step([StepEntry("a", toks_a, list(range(40)))])
    runner.end("a")
    assert _rel(got, want_a) < TOL[dtype]
    # two requests in portions and single tokens, mixed; the slot of "a" is used again (and must start from zero)
    outs = {"a": [], "b": []}
    plan = [[("a", 0, 7), ("b", 0, 2)], [("a", 7, 1), ("b", 2, 20)], [("a", 8, 31)], [("a", 39, 1), ("b", 22, 1)]]
    for step in plan:
        entries = [StepEntry(r, (toks_a if r == "a" else toks_b)[lo:lo + n], list(range(n))) for r, lo, n in step]
        logits = runner.step(entries)
        row = 0
        for r, lo, n in step:
            outs[r].append(logits[row:row + n].clone())
            row += n
    assert _rel(torch.cat(outs["a"]), want_a) < TOL[dtype]
    assert _rel(torch.cat(outs["b"]), want_b) < TOL[dtype]
    runner.end("a"), runner.end("b")
    runner.kv.check(), runner.slots.check()


# ------------------------------------ a layer twice, and a layer reading another run's cache
@pytest.mark.parametrize("dtype", DTYPES)
def test_layer_runs_twice_and_shared_cache(dtype):
    from inferflux_b200.config.spec import LayerSpec, PartSpec, Run
    from inferflux_b200.engine import StepEntry
    hidden, nh, nkv, hd = 64, 4, 2, 16
    norm = lambda name: PartSpec("rmsnorm", dict(name=name, hidden=hidden, eps=1e-6))
    shared = LayerSpec("layers.1", "prenorm", dict(
        mixer=PartSpec("gqa_attention", dict(name="attn", hidden=hidden, n_heads=nh, n_kv_heads=nkv, head_dim=hd,
                                             qkv_bias=False, o_bias=False, window=None, kv_shared=True)),
        mixer_norm=norm("n1"), feed_forward=PartSpec("swiglu", dict(name="mlp", hidden=hidden, intermediate=96)),
        feed_forward_norm=norm("n2")), position="rope")
    # run 0: layer 0; run 1: layer 1 reading run 0's keys and values; run 2: layer 0 again (a cache of its own)
    spec = _one_layer_spec(hidden, nh, nkv, hd, extra_layers=[shared], schedule=[Run(0), Run(1, cache_of=0), Run(0)])
    model, runner, w = _build(spec, dtype, 31)
    assert model.runs_per_group == [2] and [r.writes_kv for r in model.runs] == [True, False, True]
    assert "layers.1.attn.k_proj.weight" not in w and "layers.1.attn.q_proj.weight" in w

    def layer0(x, positions):
        h = plain.rms_norm(x, w["layers.0.n1.weight"], 1e-6)
        x = x + plain.attention_block(h, {k.replace("layers.0.attn", "a"): v for k, v in w.items()}, "a", positions,
                                      nh, nkv, hd, 10000.0, None)
        return x + plain.mlp_block(plain.rms_norm(x, w["layers.0.n2.weight"], 1e-6), w, "layers.0.mlp"), h

    def plain_forward(tokens):
        t = len(tokens)
        pos = torch.arange(t)
        x0 = plain.embed(w["emb.weight"], tokens)
        x, h0 = layer0(x0, pos)
        # run 0's keys and values, as they lie in its cache
        k = (h0 @ w["layers.0.attn.k_proj.weight"].T + w["layers.0.attn.k_proj.bias"]).view(t, nkv, hd)
        v = (h0 @ w["layers.0.attn.v_proj.weight"].T + w["layers.0.attn.v_proj.bias"]).view(t, nkv, hd)
        cos, sin = plain.rope_angles(pos, hd, 10000.0, torch.float64)
        k = plain.apply_rope_half(k, cos, sin)
        h = plain.rms_norm(x, w["layers.1.n1.weight"], 1e-6)
        q = plain.apply_rope_half((h @ w["layers.1.attn.q_proj.weight"].T).view(t, nh, hd), cos, sin)
        a = plain.causal_gqa_attention(q, k, v, 1.0 / math.sqrt(hd))
        x = x + a.reshape(t, nh * hd) @ w["layers.1.attn.o_proj.weight"].T
        x = x + plain.mlp_block(plain.rms_norm(x, w["layers.1.n2.weight"], 1e-6), w, "layers.1.mlp")
        x, _ = layer0(x, pos)
        return plain.rms_norm(x, w["final.weight"], 1e-6) @ w["head.weight"].T

    toks = torch.randint(0, 50, (45,), generator=torch.Generator().manual_seed(3)).tolist()
    want = plain_forward(toks)
    got = runner.step([StepEntry("w", toks, list(range(45)))])
    runner.end("w")
    assert _rel(got, want) < TOL[dtype]
    outs, pos = [], 0
    for n in (9, 2, 17, 1, 1, 15):
        outs.append(runner.step([StepEntry("c", toks[pos:pos + n], list(range(n)))]).clone())
        pos += n
    assert _rel(torch.cat(outs), want) < TOL[dtype]


# ------------------------------------------------ a toy feed-forward with routing
def _register_top2_experts():
    """A feed-forward that sends every token to its two best of E small experts
    (router logits and their softmax in float32), defined in this test."""
    from inferflux_b200.config import register_part
    from inferflux_b200.parts.base import Part
    from inferflux_b200.weights.loader import MATRIX, WeightSpec

    class Top2Experts(Part):
        family = "feed_forward"

        @classmethod
        def weight_specs(cls, params, prefix):
            h, i, e = int(params["hidden"]), int(params["intermediate"]), int(params["experts"])
            n = lambda leaf: cls.full_name(prefix, params, leaf)
            return [WeightSpec(n("router.weight"), (e, h), MATRIX, std=1.0), WeightSpec(n("up.weight"), (e * i, h), MATRIX),
                    WeightSpec(n("down.weight"), (e * h, i), MATRIX)]

        def load(self, tensors):
            n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
            e, h, i = (int(self.params[k]) for k in ("experts", "hidden", "intermediate"))
            self.router = tensors.pop(n("router.weight")).float()
            self.up = tensors.pop(n("up.weight")).float().view(e, i, h)
            self.down = tensors.pop(n("down.weight")).float().view(e, h, i)

        def forward(self, x, ctx):
            xf = x.float()
            logits = xf @ self.router.T                                   # [N, E], float32
            top, idx = torch.topk(logits, 2, dim=-1)
            gate = torch.softmax(top, dim=-1)
            out = torch.zeros_like(xf)
            for k in range(2):
                up = torch.relu(torch.einsum("nh,nih->ni", xf, self.up[idx[:, k]]))
                out += gate[:, k:k + 1] * torch.einsum("ni,nhi->nh", up, self.down[idx[:, k]])
            return out.to(x.dtype)

    register_part("feed_forward", "top2_experts", Top2Experts)


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_routed_feed_forward_is_registered_built_and_stepped(dtype):
    """One layer has the toy routed feed-forward in place of SwiGLU; nothing in
    the package knows it.  Whole, and in portions mixed with single tokens."""
    from inferflux_b200.config.spec import LayerSpec, PartSpec
    from inferflux_b200.engine import StepEntry
    _register_top2_experts()
    hidden, experts, inter = 48, 5, 24
    norm = lambda name: PartSpec("rmsnorm", dict(name=name, hidden=hidden, eps=1e-6))
    routed = LayerSpec("layers.1", "prenorm", dict(
        mixer=PartSpec("gqa_attention", dict(name="attn", hidden=hidden, n_heads=3, n_kv_heads=1, head_dim=16,
                                             qkv_bias=True, o_bias=False, window=None)), mixer_norm=norm("n1"),
        feed_forward=PartSpec("top2_experts", dict(name="moe", hidden=hidden, intermediate=inter, experts=experts)),
        feed_forward_norm=norm("n2")), position="rope")
    spec = _one_layer_spec(hidden, 3, 1, 16, extra_layers=[routed])

    def plain_forward(w, tokens):
        t = len(tokens)
        pos = torch.arange(t)
        x = plain.embed(w["emb.weight"], tokens)
        margins = []
        for layer in ("layers.0", "layers.1"):
            h = plain.rms_norm(x, w[f"{layer}.n1.weight"], 1e-6)
            ww = {k.replace(f"{layer}.attn", "a"): v for k, v in w.items()}
            x = x + plain.attention_block(h, ww, "a", pos, 3, 1, 16, 10000.0, None)
            h = plain.rms_norm(x, w[f"{layer}.n2.weight"], 1e-6)
            if layer == "layers.0":
                x = x + plain.mlp_block(h, w, "layers.0.mlp")
                continue
            logits = h @ w["layers.1.moe.router.weight"].T
            top, idx = torch.topk(logits, 3, dim=-1)
            margins.append(float((top[:, 1] - top[:, 2]).min()))
            gate = torch.softmax(top[:, :2], dim=-1)
            up_w = w["layers.1.moe.up.weight"].view(experts, inter, hidden)
            down_w = w["layers.1.moe.down.weight"].view(experts, hidden, inter)
            out = torch.zeros_like(h)
            for k in range(2):
                up = torch.relu(torch.einsum("nh,nih->ni", h, up_w[idx[:, k]]))
                out += gate[:, k:k + 1] * torch.einsum("ni,nhi->nh", up, down_w[idx[:, k]])
            x = x + out
        return plain.rms_norm(x, w["final.weight"], 1e-6) @ w["head.weight"].T, min(margins)

    # weights with which no token's second and third router logits lie close (a near tie may go
    # either way in bfloat16, and then the comparison would say nothing about the engine)
    toks = torch.randint(0, 50, (37,), generator=torch.Generator().manual_seed(5)).tolist()
    for seed in range(40, 140):
        model, runner, w = _build(spec, dtype, seed)
        want, margin = plain_forward(w, toks)
        if margin > 0.3:                                 # router logits are of the order of 7 here
            break
    else:
        pytest.fail("no seed with a clear routing margin")
    got = runner.step([StepEntry("w", toks, list(range(37)))])
    runner.end("w")
    assert _rel(got, want) < TOL[dtype]
    outs, pos = [], 0
    for n in (5, 1, 1, 20, 2, 8):
        outs.append(runner.step([StepEntry("c", toks[pos:pos + n], list(range(n)))]).clone())
        pos += n
    assert _rel(torch.cat(outs), want) < TOL[dtype]


# ------------------------------------------------ a toy position encoding
def _register_learned_rotary():
    """Rotary positions whose frequencies are a weight of the model (one per pair
    of dims) instead of a power law, defined in this test.  The attention part
    takes its (cos, sin) as it takes the built-in ones."""
    from inferflux_b200.config import register_part
    from inferflux_b200.parts.base import Part
    from inferflux_b200.weights.loader import VECTOR, WeightSpec

    class LearnedRotary(Part):
        family = "position"

        @classmethod
        def weight_specs(cls, params, prefix):
            return [WeightSpec(cls.full_name(prefix, params, "freq"), (int(params["rotary_dim"]) // 2,), VECTOR, std=0.3)]

        def load(self, tensors):
            self.freq = tensors.pop(self.full_name(self.prefix, self.params, "freq")).double()

        def prepare(self, ctx):
            a = ctx.positions.double()[:, None] * self.freq[None, :]
            return torch.cos(a).float(), torch.sin(a).float()

    register_part("position", "learned_rotary", LearnedRotary)


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_position_encoding_is_registered_built_and_stepped(dtype):
    from inferflux_b200.config.spec import LayerSpec, ModelSpec, PartSpec, Run
    from inferflux_b200.engine import StepEntry
    _register_learned_rotary()
    hidden, nh, nkv, hd = 64, 4, 2, 16
    spec = _one_layer_spec(hidden, nh, nkv, hd)
    spec.positions["rope"] = PartSpec("learned_rotary", dict(name="pos", rotary_dim=hd))
    model, runner, w = _build(spec, dtype, 77)
    assert "pos.freq" in w

    def plain_forward(tokens):
        t = len(tokens)
        x = plain.embed(w["emb.weight"], tokens)
        h = plain.rms_norm(x, w["layers.0.n1.weight"], 1e-6)
        a = torch.arange(t, dtype=torch.float64)[:, None] * w["pos.freq"][None, :]
        cos, sin = torch.cos(a), torch.sin(a)
        p = "layers.0.attn"
        q = plain.apply_rope_half((h @ w[f"{p}.q_proj.weight"].T + w[f"{p}.q_proj.bias"]).view(t, nh, hd), cos, sin)
        k = plain.apply_rope_half((h @ w[f"{p}.k_proj.weight"].T + w[f"{p}.k_proj.bias"]).view(t, nkv, hd), cos, sin)
        v = (h @ w[f"{p}.v_proj.weight"].T + w[f"{p}.v_proj.bias"]).view(t, nkv, hd)
        x = x + plain.causal_gqa_attention(q, k, v, 1.0 / math.sqrt(hd)).reshape(t, nh * hd) @ w[f"{p}.o_proj.weight"].T
        x = x + plain.mlp_block(plain.rms_norm(x, w["layers.0.n2.weight"], 1e-6), w, "layers.0.mlp")
        return plain.rms_norm(x, w["final.weight"], 1e-6) @ w["head.weight"].T

    toks = torch.randint(0, 50, (41,), generator=torch.Generator().manual_seed(6)).tolist()
    want = plain_forward(toks)
    got = runner.step([StepEntry("w", toks, list(range(41)))])
    runner.end("w")
    assert _rel(got, want) < TOL[dtype]
    outs, pos = [], 0
    for n in (3, 30, 1, 1, 6):
        outs.append(runner.step([StepEntry("c", toks[pos:pos + n], list(range(n)))]).clone())
        pos += n
    assert _rel(torch.cat(outs), want) < TOL[dtype]


# ------------------------- a block with four norms around a mixer that caches one latent vector per token
def _register_sandwich_and_latent():
    """Two toys defined in this test.  ``sandwich``: an arrangement with a norm
    before and a norm after each branch, so six roles instead of four.
    ``latent_attention``: a mixer that keeps one vector of ``latent`` elements
    per token in the paged cache (a single stream, no keys and values) and
    attends over those vectors."""
    from inferflux_b200.config import register_part
    from inferflux_b200.parts.base import CacheStream, KVNeed, Part, PartialSums
    from inferflux_b200.weights.loader import MATRIX, WeightSpec

    def dense(y):
        return y.tensor.sum(0) if isinstance(y, PartialSums) else y.float()

    class SandwichBlock:
        family = "arrangement"
        roles = {"mixer": "mixer", "mixer_norm": "norm", "mixer_post_norm": "norm", "feed_forward": "feed_forward",
                 "feed_forward_norm": "norm", "feed_forward_post_norm": "norm"}
        optional_roles = frozenset()

        def __init__(self, parts, position_name):
            self.p, self.position_name = parts, position_name

        def forward(self, residual, delta, ctx, run):
            p = self.p
            x = p["mixer_norm"].forward(residual, delta)
            position = ctx.position_tables.get(self.position_name) if self.position_name else None
            a = p["mixer_post_norm"].forward(dense(p["mixer"].forward(x, ctx, run, position)), None)
            x2 = p["feed_forward_norm"].forward(residual, a)
            return p["feed_forward_post_norm"].forward(dense(p["feed_forward"].forward(x2, ctx)), None)

    class LatentAttention(Part):
        family = "mixer"

        @classmethod
        def weight_specs(cls, params, prefix):
            h, l = int(params["hidden"]), int(params["latent"])
            n = lambda leaf: cls.full_name(prefix, params, leaf)
            return [WeightSpec(n("down.weight"), (l, h), MATRIX, std=0.3), WeightSpec(n("up.weight"), (h, l), MATRIX, std=0.3)]

        @classmethod
        def kv_need(cls, params):
            return KVNeed((CacheStream("latent", 1, int(params["latent"])),), None)

        def load(self, tensors):
            n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
            self.down, self.up = tensors.pop(n("down.weight")).float(), tensors.pop(n("up.weight")).float()

        def forward(self, x, ctx, run, position):
            g, ps, l = run.kv_group, ctx.page_size, int(self.params["latent"])
            views, stride = ctx.kv.stream_views(g, run.kv_index)
            pool = ctx.kv.pools[g]
            cache = torch.as_strided(pool, (pool.shape[0], ps, l), (stride, l, 1), views["latent"].storage_offset())
            slots = ctx.slot_maps[g].long()
            cache[slots // ps, slots % ps] = (x.float() @ self.down.T).to(cache.dtype)
            out = torch.empty((x.shape[0], self.up.shape[0]), dtype=torch.float32, device=x.device)
            row = 0
            for e, (entry, start) in enumerate(zip(ctx.entries, ctx.ctx_starts)):
                n, total = len(entry.tokens), start + len(entry.tokens)
                table = ctx.block_tables[g][e, :(total + ps - 1) // ps].long()
                lat = cache[table].reshape(-1, l)[:total].float()
                s = lat[start:] @ lat.T / math.sqrt(l)
                keys = torch.arange(total, device=x.device)[None, :]
                s = s.masked_fill(keys > torch.arange(start, total, device=x.device)[:, None], float("-inf"))
                out[row:row + n] = torch.softmax(s, -1) @ lat @ self.up.T
                row += n
            return out.to(x.dtype)

    register_part("arrangement", "sandwich", SandwichBlock)
    register_part("mixer", "latent_attention", LatentAttention)


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_block_with_four_norms_and_a_latent_cache(dtype):
    from inferflux_b200.config.spec import LayerSpec, PartSpec
    from inferflux_b200.engine import StepEntry
    _register_sandwich_and_latent()
    hidden, latent = 64, 24
    norm = lambda name: PartSpec("rmsnorm", dict(name=name, hidden=hidden, eps=1e-6))
    toy = LayerSpec("layers.1", "sandwich", dict(
        mixer=PartSpec("latent_attention", dict(name="lat", hidden=hidden, latent=latent)), mixer_norm=norm("n1"),
        mixer_post_norm=norm("p1"), feed_forward=PartSpec("swiglu", dict(name="mlp", hidden=hidden, intermediate=96)),
        feed_forward_norm=norm("n2"), feed_forward_post_norm=norm("p2")), position=None)
    spec = _one_layer_spec(hidden, 4, 2, 16, extra_layers=[toy])
    # a layer that lists a role its arrangement does not have, or lacks one, is refused with both named
    from inferflux_b200.engine import Model
    import dataclasses
    bad = dataclasses.replace(toy, arrangement="prenorm")
    with pytest.raises(ValueError, match="mixer_post_norm"):
        Model(_one_layer_spec(hidden, 4, 2, 16, extra_layers=[bad]), dtype, DEV)
    model, runner, w = _build(spec, dtype, 91)
    # two cache groups: keys and values of layer 0, one latent vector a token of layer 1
    assert [[s.name for s in n.streams] for n in model.kv_needs] == [["k", "v"], ["latent"]]
    assert runner.kv_storage.pools[1].shape[2] == 16 * latent and "layers.1.p2.weight" in w

    def plain_forward(tokens):
        t = len(tokens)
        x = plain.embed(w["emb.weight"], tokens)
        h = plain.rms_norm(x, w["layers.0.n1.weight"], 1e-6)
        x = x + plain.attention_block(h, {k.replace("layers.0.attn", "a"): v for k, v in w.items()}, "a",
                                      torch.arange(t), 4, 2, 16, 10000.0, None)
        x = x + plain.mlp_block(plain.rms_norm(x, w["layers.0.n2.weight"], 1e-6), w, "layers.0.mlp")
        c = plain.rms_norm(x, w["layers.1.n1.weight"], 1e-6) @ w["layers.1.lat.down.weight"].T
        s = (c @ c.T / math.sqrt(latent)).masked_fill(torch.arange(t)[None, :] > torch.arange(t)[:, None], float("-inf"))
        a = torch.softmax(s, -1) @ c @ w["layers.1.lat.up.weight"].T
        x = x + plain.rms_norm(a, w["layers.1.p1.weight"], 1e-6)
        f = plain.mlp_block(plain.rms_norm(x, w["layers.1.n2.weight"], 1e-6), w, "layers.1.mlp")
        x = x + plain.rms_norm(f, w["layers.1.p2.weight"], 1e-6)
        return plain.rms_norm(x, w["final.weight"], 1e-6) @ w["head.weight"].T

    toks_a = torch.randint(0, 50, (40,), generator=torch.Generator().manual_seed(11)).tolist()
    toks_b = torch.randint(0, 50, (23,), generator=torch.Generator().manual_seed(12)).tolist()
    want_a, want_b = plain_forward(toks_a), plain_forward(toks_b)
    got = runner.step([StepEntry("w", toks_a, list(range(40)))])
    runner.end("w")
    assert _rel(got, want_a) < TOL[dtype]
    outs = {"a": [], "b": []}
    plan = [[("a", 0, 7), ("b", 0, 2)], [("a", 7, 1), ("b", 2, 20)], [("a", 8, 31)], [("a", 39, 1), ("b", 22, 1)]]
    for step in plan:
        entries = [StepEntry(r, (toks_a if r == "a" else toks_b)[lo:lo + n], list(range(n))) for r, lo, n in step]
        logits = runner.step(entries)
        row = 0
        for r, lo, n in step:
            outs[r].append(logits[row:row + n].clone())
            row += n
    assert _rel(torch.cat(outs["a"]), want_a) < TOL[dtype]
    assert _rel(torch.cat(outs["b"]), want_b) < TOL[dtype]
    runner.end("a"), runner.end("b")
    runner.kv.check()
