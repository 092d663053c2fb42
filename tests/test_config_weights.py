"""Configuration, registry, safetensors and weight binding (no GPU)."""
from __future__ import annotations

import json
import os
import struct

import pytest
import torch

from helpers import TINY_A, TINY_B, TINY_E, make_model_folder
from inferflux_b200.config import (ConfigError, Qwen2Config, build_spec, load_config, register_architecture,
                                   registered_architectures, resolve_architecture)
from inferflux_b200.config.spec import LayerSpec, ModelSpec, PartSpec, Run
from inferflux_b200.engine.model import Model
from inferflux_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError, load_weights,
                                    write_safetensors)
from inferflux_b200.weights.random_init import random_tensors, write_random_model


def test_config_reads_every_key():
    c = Qwen2Config.from_dict(TINY_E)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (96, 3, 3, 1, 32)
    assert (c.intermediate_size, c.vocab_size, c.max_position_embeddings) == (256, 1000, 512)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and not c.tie_word_embeddings
    assert [c.window_of_layer(i) for i in range(3)] == [None, 40, 40]
    a = Qwen2Config.from_dict(TINY_A)
    assert a.tie_word_embeddings and [a.window_of_layer(i) for i in range(2)] == [None, None]
    assert [Qwen2Config.from_dict(TINY_B).window_of_layer(i) for i in range(3)] == [None, None, None]


def test_config_defaults_and_errors():
    d = dict(TINY_A)
    del d["head_dim"], d["num_key_value_heads"], d["rope_theta"], d["rms_norm_eps"]
    c = Qwen2Config.from_dict(d)
    assert c.head_dim == 16 and c.num_key_value_heads == 4 and c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-6
    for key in ("hidden_size", "num_hidden_layers", "intermediate_size", "vocab_size", "max_position_embeddings"):
        bad = dict(TINY_A)
        del bad[key]
        with pytest.raises(ConfigError, match=key):
            Qwen2Config.from_dict(bad)
    with pytest.raises(ConfigError, match="multiple"):
        Qwen2Config.from_dict(dict(TINY_A, num_key_value_heads=3))
    with pytest.raises(ConfigError, match="hidden_act"):
        Qwen2Config.from_dict(dict(TINY_A, hidden_act="gelu"))
    with pytest.raises(ConfigError, match="rope_scaling"):
        Qwen2Config.from_dict(dict(TINY_A, rope_scaling={"type": "yarn", "factor": 4}))
    with pytest.raises(ConfigError, match="sliding_window"):
        Qwen2Config.from_dict(dict(TINY_A, use_sliding_window=True))
    with pytest.raises(ConfigError, match="integer"):
        Qwen2Config.from_dict(dict(TINY_A, hidden_size="64"))


def test_registry_by_architecture_or_model_type():
    assert "Qwen2ForCausalLM" in registered_architectures()
    assert resolve_architecture({"architectures": ["Qwen2ForCausalLM"]}) == "Qwen2ForCausalLM"
    assert resolve_architecture({"model_type": "Qwen2"}) == "Qwen2ForCausalLM"      # the reference's key
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})


def test_spec_is_data_per_layer():
    spec = build_spec(Qwen2Config.from_dict(TINY_E))
    assert len(spec.layers) == 3 and [r.layer for r in spec.schedule] == [0, 1, 2]
    assert [l.part("mixer").params["window"] for l in spec.layers] == [None, 40, 40]
    assert spec.layers[0].part("mixer").kind == "gqa_attention" and spec.layers[0].part("feed_forward").kind == "swiglu"
    assert sorted(spec.layers[0].parts) == ["feed_forward", "feed_forward_norm", "mixer", "mixer_norm"]
    m = Model(spec, torch.float32, "cpu")
    # layers with and without a window are cache groups of their own
    assert [n.window for n in m.kv_needs] == [None, 40] and m.runs_per_group == [1, 2]
    names = {w.name for w in m.weight_specs()}
    assert "model.layers.2.self_attn.q_proj.bias" in names and "lm_head.weight" in names
    assert "model.layers.0.self_attn.o_proj.bias" not in names


def test_schedule_validation():
    spec = build_spec(Qwen2Config.from_dict(TINY_A))
    spec.schedule = [Run(0), Run(1), Run(1)]            # a layer twice: allowed
    spec.validate()
    m = Model(spec, torch.float32, "cpu")
    assert m.runs_per_group == [3]                      # each run has a cache of its own
    spec.schedule = [Run(0), Run(5)]
    with pytest.raises(ValueError, match="layer 5"):
        spec.validate()
    spec.schedule = [Run(0, cache_of=0)]
    with pytest.raises(ValueError, match="earlier"):
        spec.validate()
    spec.schedule = [Run(0), Run(1, cache_of=0)]        # layer 1 has k/v of its own: not allowed to share
    with pytest.raises(ValueError, match="keys and values of its own"):
        Model(spec, torch.float32, "cpu")


def test_safetensors_roundtrip_and_format(tmp_path):
    t = {"a.weight": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int32),
         "c": torch.randn(4), "empty": torch.zeros(0, 3)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t, metadata={"format": "pt"})
    raw = open(path, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    assert header["a.weight"] == {"dtype": "BF16", "shape": [3, 5], "data_offsets": [0, 30]}
    assert (8 + hlen) % 8 == 0 and "__metadata__" in header
    f = SafetensorsFile(path)
    assert sorted(f.names()) == sorted(t)
    for k, v in t.items():
        got = f.tensor(k)
        assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v)
    f.close()
    # the safetensors library reads the same file
    from safetensors import safe_open
    with safe_open(path, framework="pt") as g:
        assert torch.equal(g.get_tensor("a.weight"), t["a.weight"])


def test_safetensors_faults(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    open(p, "wb").write(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 12)
    with pytest.raises(SafetensorsError, match="12 bytes but shape"):
        SafetensorsFile(p)
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    open(p, "wb").write(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)          # truncated data
    with pytest.raises(SafetensorsError, match="outside the data"):
        SafetensorsFile(p)


def test_weight_errors_list_everything(tmp_path):
    folder = make_model_folder(TINY_A, 0, str(tmp_path / "m"))
    spec = build_spec(load_config(folder))
    model = Model(spec, torch.float32, "cpu")
    good = load_weights(folder, model.weight_specs(), torch.float32, "cpu")
    assert len(good) == 2 * 12 + 2
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.tensor(n) for n in f.names()}
    f.close()
    del tensors["model.layers.1.mlp.up_proj.weight"], tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63, dtype=torch.bfloat16)
    tensors["model.layers.7.extra.weight"] = torch.zeros(2)
    tensors["rotary.inv_freq"] = torch.zeros(8)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with pytest.raises(WeightsError) as ei:
        load_weights(folder, model.weight_specs(), torch.float32, "cpu")
    e = ei.value
    assert sorted(e.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.7.extra.weight", "rotary.inv_freq"]
    assert e.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (64, 63), (64, 64))]
    msg = str(e)
    for piece in ("missing (2)", "unexpected (2)", "wrong shape (1)", "is [64, 63], expected [64, 64]"):
        assert piece in msg


def test_tied_head_ignores_a_stored_lm_head(tmp_path):
    folder = make_model_folder(TINY_A, 0, str(tmp_path / "m"))
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.tensor(n) for n in f.names()}
    f.close()
    assert "lm_head.weight" not in tensors
    tensors["lm_head.weight"] = torch.zeros(512, 64, dtype=torch.bfloat16)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    model = Model(build_spec(load_config(folder)), torch.float32, "cpu")
    loaded = load_weights(folder, model.weight_specs(), torch.float32, "cpu")
    assert "lm_head.weight" not in loaded


def test_storage_dtypes(tmp_path):
    folder = make_model_folder(TINY_B, 1, str(tmp_path / "m"), vector_dtype=torch.float32)
    model = Model(build_spec(load_config(folder)), torch.bfloat16, "cpu")
    bf = load_weights(folder, model.weight_specs(), torch.bfloat16, "cpu")
    assert bf["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16     # 16-bit stays bfloat16
    assert bf["model.norm.weight"].dtype == torch.float32                       # stored in 32-bit stays so
    f32 = load_weights(folder, model.weight_specs(), torch.float32, "cpu")
    assert f32["model.layers.0.mlp.down_proj.weight"].dtype == torch.float32
    assert torch.equal(f32["model.layers.0.mlp.down_proj.weight"], bf["model.layers.0.mlp.down_proj.weight"].float())


def test_sharded_folder(tmp_path):
    folder = make_model_folder(TINY_A, 0, str(tmp_path / "m"))
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.tensor(n) for n in f.names()}
    f.close()
    os.remove(os.path.join(folder, "model.safetensors"))
    names = sorted(tensors)
    half = len(names) // 2
    write_safetensors(os.path.join(folder, "model-00001-of-00002.safetensors"), {n: tensors[n] for n in names[:half]})
    write_safetensors(os.path.join(folder, "model-00002-of-00002.safetensors"), {n: tensors[n] for n in names[half:]})
    wm = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
          for i, n in enumerate(names)}
    json.dump({"weight_map": wm}, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    model = Model(build_spec(load_config(folder)), torch.float32, "cpu")
    assert len(load_weights(folder, model.weight_specs(), torch.float32, "cpu")) == len(names)
    os.remove(os.path.join(folder, "model-00002-of-00002.safetensors"))
    with pytest.raises(SafetensorsError, match="missing"):
        load_weights(folder, model.weight_specs(), torch.float32, "cpu")


def test_random_model_folder_is_seeded(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_A)
    a, b, c = (write_random_model(str(tmp_path / n), cfg, s) for n, s in (("a", 5), ("b", 5), ("c", 6)))
    ra = open(os.path.join(a, "model.safetensors"), "rb").read()
    assert ra == open(os.path.join(b, "model.safetensors"), "rb").read()
    assert ra != open(os.path.join(c, "model.safetensors"), "rb").read()
    assert load_config(a) == cfg
    f = SafetensorsFile(os.path.join(a, "model.safetensors"))
    w = f.tensor("model.layers.0.mlp.gate_proj.weight").float()
    n = f.tensor("model.norm.weight").float()
    f.close()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.001
    assert abs(float(n.mean()) - 1.0) < 0.02


def test_another_architecture_can_be_registered():
    """A made-up architecture name mapped to a spec built from the same parts."""
    from dataclasses import dataclass
    from inferflux_b200.config.model_config import ModelConfig

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        width: int = 32

        @classmethod
        def from_dict(cls, d):
            return cls(architectures=list(d["architectures"]), width=int(d["width"]))

    def build(cfg):
        norm = lambda name: PartSpec("rmsnorm", dict(name=name, hidden=cfg.width, eps=1e-5))
        layer = LayerSpec("blocks.0", "prenorm", dict(
            mixer=PartSpec("gqa_attention", dict(name="attn", hidden=cfg.width, n_heads=2, n_kv_heads=1,
                                                 head_dim=16, qkv_bias=False, o_bias=True, window=None)),
            mixer_norm=norm("n1"), feed_forward=PartSpec("swiglu", dict(name="ff", hidden=cfg.width, intermediate=48)),
            feed_forward_norm=norm("n2")), position=None)
        return ModelSpec("ToyLM", cfg.width, 50, 64, PartSpec("token_embedding", dict(name="emb", vocab=50, hidden=cfg.width)),
                         norm("final"), PartSpec("linear_head", dict(name="head", vocab=50, hidden=cfg.width, tied_to=None)),
                         {}, [layer], [Run(0)])

    register_architecture("ToyLM", ToyConfig, build)
    cfg = load_config({"architectures": ["ToyLM"], "width": 32})
    m = Model(build_spec(cfg), torch.float32, "cpu")
    names = {w.name for w in m.weight_specs()}
    assert {"blocks.0.attn.o_proj.bias", "blocks.0.ff.down_proj.weight", "emb.weight", "head.weight"} <= names
    assert "blocks.0.attn.q_proj.bias" not in names
