"""The engine at the layer sizes of a real model of the family (Qwen2.5-7B:
hidden 3584, 28 query heads on 4 key/value heads of size 128, feed-forward
18944, vocabulary 152064), cut to two layers so that the plain implementation
can follow on the CPU.  At these sizes the engine takes the paths the tiny
models never reach: the tcgen05 attention and product kernels for prompt
portions, the planned K splits of the weight-streaming product, decode
attention split over the keys, argmax over a wide vocabulary."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from helpers import TOL, random_tokens

pytestmark = pytest.mark.gpu

FAMILY = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=3584, num_hidden_layers=2,
              num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944,
              vocab_size=152064, max_position_embeddings=4096, rope_theta=1e6, rms_norm_eps=1e-6,
              tie_word_embeddings=False, use_sliding_window=False)


@pytest.fixture(scope="module")
def family():
    """Random bfloat16 weights made on the CPU: the engine gets them as they are,
    the plain implementation as float32."""
    from inferflux_b200 import Engine
    from inferflux_b200.config import EngineConfig, load_config
    from inferflux_b200.config.registry import build_spec
    from inferflux_b200.engine.model import Model
    from inferflux_b200.weights.random_init import random_tensors
    config = load_config(dict(FAMILY))
    ecfg = EngineConfig(dtype="bfloat16", kv_cache_tokens=2048, max_seqs=4, max_batch_tokens=1024,
                        chunked_prefill_tokens=512)
    model = Model(build_spec(config), torch.bfloat16, ecfg.device)
    tensors = random_tensors(model.weight_specs(), 7, torch.bfloat16, torch.float32, "cpu")
    w = {k: v.float() for k, v in tensors.items()}
    model.load({k: v.to(ecfg.device) for k, v in tensors.items()})
    del tensors
    return Engine(model, config, ecfg), dict(FAMILY), w


def _check(got, hidden, head, rows, what):
    want = hidden[rows] @ head.T
    err = float((got.double().cpu() - want.double()).abs().max() / want.abs().max())
    assert err <= TOL["bfloat16"], f"{what}: {err:.3e}"
    return want


def test_prompts_then_decoding_at_family_sizes(family):
    from inferflux_b200 import SamplingParams, StepEntry
    eng, cfg, w = family
    torch.set_num_threads(max(1, torch.get_num_threads()))
    a = random_tokens(cfg["vocab_size"], 308, 201)
    b = random_tokens(cfg["vocab_size"], 158, 202)
    head = plain.head_weight(cfg, w)
    ha, hb = plain.final_hidden(cfg, w, a), plain.final_hidden(cfg, w, b)
    # two prompt portions in one step (450 rows: tcgen05 product and attention), logits at three places
    logits = eng.run_step([StepEntry("a", a[:300], [0, 299]), StepEntry("b", b[:150], [149])])
    _check(logits[:2], ha, head, [0, 299], "prompt a")
    _check(logits[2:], hb, head, [149], "prompt b")
    # eight tokens one at a time, both requests side by side (captured decode steps, weight-streaming products)
    for i in range(8):
        logits = eng.run_step([StepEntry("a", [a[300 + i]], [0]), StepEntry("b", [b[150 + i]], [0])])
        want_a = _check(logits[:1], ha, head, [300 + i], f"decode a {i}")
        _check(logits[1:], hb, head, [150 + i], f"decode b {i}")
        # the device's argmax over the wide vocabulary
        ids = eng.sampler.sample(logits.clone(), [SamplingParams(temperature=0.0)] * 2, [0, 0], [0, 0], [(), ()])
        assert int(ids[0]) == int(torch.argmax(logits[0])) and int(ids[1]) == int(torch.argmax(logits[1]))
        top = float(want_a.max())
        assert float(want_a[0, int(ids[0])]) >= top - 2 * TOL["bfloat16"] * float(want_a.abs().max())
    assert eng.runner.graph_replays >= 4                  # two eager steps, the capture, then replays
    eng.end_request("a")
    eng.end_request("b")
    # a prompt in portions of 128 and 172 tokens gives the same logits as whole
    first = eng.run_step([StepEntry("c", a[:128], [])])
    logits = eng.run_step([StepEntry("c", a[128:300], [171])])
    _check(logits, ha, head, [299], "prompt a in two portions")
    eng.end_request("c")
    assert eng.stats["pages_free"] == eng.stats["pages_total"]
