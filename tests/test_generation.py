"""Generation through the Python entry point against the plain implementation:
greedy continuations, long decoding token by token (captured decode steps),
the first tokens of a sequence, temperature sampling that does not depend on
the batch, preemption when pages run out, penalties."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from helpers import TINY, TOL, make_model_folder, random_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders():
    out = {}
    for name in ("A", "B", "D", "E"):
        folder = make_model_folder(TINY[name], seed=40 + ord(name), sharpen=4.0)
        out[name] = (folder, *plain.load_folder(folder))
    return out


def _engine(folder, dtype, **kw):
    from inferflux_b200 import Engine
    opts = dict(kv_cache_tokens=1024, max_seqs=8)
    opts.update(kw)
    return Engine.from_pretrained(folder, dtype=dtype, **opts)


def _check_greedy(cfg, w, prompt, tokens, dtype):
    """Every generated token is the plain implementation's argmax given the
    tokens before it (bfloat16: within the tolerance of the largest logit)."""
    seq = list(prompt)
    for t in tokens:
        logits = plain.forward(cfg, w, seq)[-1]
        if dtype == "float32":
            assert t == int(torch.argmax(logits)), (len(seq), t)
        else:
            assert float(logits.max() - logits[t]) <= 2 * TOL[dtype] * float(logits.abs().max()), (len(seq), t)
        seq.append(t)


def _same_tokens(cfg, w, prompt, sp, want, got, dtype):
    """The two runs gave the same tokens.  In bfloat16 two schedules round differently (a token's keys come
    from another product when its request starts again), so a greedy request may part ways where the plain
    implementation's two best logits, penalties applied, lie within the tolerance of each other: then both
    tokens must be among those, and what follows is no longer compared."""
    if want == got:
        return
    assert dtype == "bfloat16" and sp.temperature == 0.0, (want, got)
    j = next(i for i, (a, b) in enumerate(zip(want, got)) if a != b)
    seq = list(prompt) + list(want[:j])
    logits = plain.apply_penalties(plain.forward(cfg, w, seq)[-1], seq[-sp.penalty_last_n:], sp.repetition_penalty,
                                   sp.frequency_penalty, sp.presence_penalty)
    for t in (want[j], got[j]):
        assert float(logits.max() - logits[t]) <= 2 * TOL[dtype] * float(logits.abs().max()), (j, t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D", "E"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    from inferflux_b200 import SamplingParams
    folder, cfg, w = folders[name]
    lengths = [5, 17, 33] if name == "A" else [1, 9, 40, 70]
    prompts = [random_tokens(cfg["vocab_size"], n, 60 + n) for n in lengths]
    eng = _engine(folder, dtype, chunked_prefill_tokens=16, max_batch_tokens=48)
    res = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True))
    assert [r.finish_reason for r in res] == ["length"] * len(prompts)
    for p, r in zip(prompts, res):
        assert len(r.tokens) == 16 and r.prompt_tokens == len(p)
        _check_greedy(cfg, w, p, r.tokens, dtype)
    assert eng.stats["pages_free"] == eng.stats["pages_total"]
    if dtype == "bfloat16":
        assert eng.runner.graph_replays > 0          # decode-only steps ran as captured graphs


def test_generate_leaves_the_collector_as_it_found_it(folders):
    """Engine.generate holds the cycle collector off while it steps and puts it back, also when a step raises."""
    import gc
    from inferflux_b200 import SamplingParams
    folder, cfg, _ = folders["A"]
    eng = _engine(folder, "bfloat16")
    seen = []
    step = eng.step
    eng.step = lambda: (seen.append(gc.isenabled()), step())[1]
    assert gc.isenabled()
    eng.generate([random_tokens(cfg["vocab_size"], 7, 3)], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    assert seen and not any(seen) and gc.isenabled()

    def broken():
        raise RuntimeError("a step that fails")
    eng.step = broken
    with pytest.raises(RuntimeError):
        eng.generate([random_tokens(cfg["vocab_size"], 7, 4)], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    assert gc.isenabled()
    gc.disable()
    try:
        eng.step = step
        eng.generate([random_tokens(cfg["vocab_size"], 7, 5)], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))
        assert not gc.isenabled()                            # it was off before: it stays off
    finally:
        gc.enable()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_long_decoding_token_by_token(folders, name, dtype):
    """Two prompt tokens, then 200 tokens one at a time (three requests side by
    side, crossing a dozen page borders and, in D, the window); the logits of
    every step are compared."""
    from inferflux_b200 import StepEntry
    folder, cfg, w = folders[name]
    n = 200
    seqs = [random_tokens(cfg["vocab_size"], n, 70 + i) for i in range(3)]
    refs = [plain.forward(cfg, w, s).numpy() for s in seqs]
    eng = _engine(folder, dtype)
    got = [[] for _ in seqs]
    first = eng.run_step([StepEntry(f"r{i}", s[:2], [0, 1]) for i, s in enumerate(seqs)]).cpu().numpy()
    for i in range(3):
        got[i] += [first[2 * i], first[2 * i + 1]]
    for p in range(2, n):
        logits = eng.run_step([StepEntry(f"r{i}", [s[p]], [0]) for i, s in enumerate(seqs)]).cpu().numpy()
        for i in range(3):
            got[i].append(logits[i])
    for i in range(3):
        err = np.abs(np.stack(got[i]).astype(np.float64) - refs[i]).max() / np.abs(refs[i]).max()
        assert err <= TOL[dtype], f"request {i}: {err:.3e}"
    assert eng.runner.graph_replays >= n - 8             # all but the first steps of the shape and its capture


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(folders, dtype):
    """Position 0 alone, positions 0-1, and a one-token prompt beside longer ones."""
    from inferflux_b200 import StepEntry
    folder, cfg, w = folders["E"]
    a, b, c = (random_tokens(cfg["vocab_size"], n, 80 + n) for n in (1, 2, 19))
    eng = _engine(folder, dtype)
    logits = eng.run_step([StepEntry("a", a, [0]), StepEntry("b", b, [0, 1]), StepEntry("c", c, [0, 18])]).cpu().double()
    want = torch.cat([plain.forward(cfg, w, a), plain.forward(cfg, w, b), plain.forward(cfg, w, c)[[0, 18]]])
    assert float((logits - want).abs().max() / want.abs().max()) <= TOL[dtype]
    # the first token's logits do not depend on what follows it
    assert float((logits[1] - plain.forward(cfg, w, b[:1])[0]).abs().max() / want.abs().max()) <= TOL[dtype]


def test_sampling_does_not_depend_on_the_batch(folders):
    from inferflux_b200 import SamplingParams
    folder, cfg, w = folders["A"]
    prompts = [random_tokens(cfg["vocab_size"], n, 90 + n) for n in (4, 11, 26)]
    params = [SamplingParams(temperature=0.8, seed=7 + i, max_tokens=24, ignore_eos=True, top_p=0.95) for i in range(3)]
    together = _engine(folder, "float32").generate(prompts, params)
    for i in range(3):
        alone = _engine(folder, "float32", chunked_prefill_tokens=5).generate([prompts[i]], [params[i]])
        assert alone[0].tokens == together[i].tokens
    # another seed gives another continuation; the same seed the same one
    other = _engine(folder, "float32").generate([prompts[0]], SamplingParams(temperature=0.8, seed=1234, max_tokens=24,
                                                                            ignore_eos=True, top_p=0.95))
    assert other[0].tokens != together[0].tokens
    # every sampled token lies in the plain implementation's nucleus
    seq = list(prompts[0])
    for t in together[0].tokens:
        kept = plain.kept_probabilities(plain.forward(cfg, w, seq)[-1], 0.8, 0, 0.95, 0.0)
        assert kept[t] > 0
        seq.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_when_pages_run_out_keeps_the_output(folders, dtype):
    from inferflux_b200 import SamplingParams
    folder, cfg, w = folders["A"]
    prompts = [random_tokens(cfg["vocab_size"], n, 100 + n) for n in (30, 28, 9, 33)]
    sp = SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True)
    roomy = _engine(folder, dtype).generate(prompts, sp)
    tight_engine = _engine(folder, dtype, kv_cache_tokens=112, max_seqs=4, chunked_prefill_tokens=16, max_batch_tokens=40)
    tight = tight_engine.generate(prompts, sp)
    assert tight_engine.stats["preemptions"] > 0 and sum(r.preemptions for r in tight) > 0
    for p, a, b in zip(prompts, roomy, tight):
        assert b.finish_reason == "length" and len(b.tokens) == 30
        if dtype == "float32":
            assert a.tokens == b.tokens
        _check_greedy(cfg, w, p, b.tokens, dtype)
    assert tight_engine.stats["pages_free"] == tight_engine.stats["pages_total"]
    assert sum(tight_engine.stats["page_reuses"]) > 0


def test_penalties_and_stop(folders):
    from inferflux_b200 import SamplingParams
    folder, cfg, w = folders["A"]
    prompt = random_tokens(cfg["vocab_size"], 12, 111)
    plain_logits = plain.forward(cfg, w, prompt)[-1]
    first = int(torch.argmax(plain_logits))
    # a presence penalty on a prompt made of the would-be winner pushes it out
    pen = SamplingParams(temperature=0.0, max_tokens=1, presence_penalty=100.0, repetition_penalty=1.3, ignore_eos=True)
    prompt2 = prompt[:-1] + [first]
    want = plain.apply_penalties(plain.forward(cfg, w, prompt2)[-1], prompt2[-pen.penalty_last_n:], 1.3, 0.0, 100.0)
    got = _engine(folder, "float32").generate([prompt2], pen)[0].tokens
    assert got == [int(torch.argmax(want))] and got[0] not in prompt2
    # stop tokens end a request early
    stop = SamplingParams(temperature=0.0, max_tokens=20, stop_token_ids=[first], ignore_eos=True)
    r = _engine(folder, "float32").generate([prompt], stop)[0]
    assert r.tokens == [first] and r.finish_reason == "stop"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_queued_behind_a_busy_gpu(folders, dtype):
    """The host may prepare several steps while the GPU still works on an
    earlier one: each step's metadata must survive until its kernels have read
    it.  A long library product keeps the GPU busy while six different steps
    are queued without any synchronisation."""
    from inferflux_b200 import StepEntry
    folder, cfg, w = folders["A"]
    eng = _engine(folder, dtype, cuda_graphs=False)
    seqs = [random_tokens(cfg["vocab_size"], n, 120 + n) for n in (90, 37, 64, 130, 5, 71)]
    busy = torch.randn(8192, 8192, device="cuda:0")
    for _ in range(40):
        busy = (busy @ busy).clamp_(-1, 1)
    outs = []
    for i, s in enumerate(seqs):                    # no synchronisation between these steps
        half = max(1, len(s) // 2)
        eng.run_step([StepEntry(f"q{i}", s[:half], [])])
        outs.append(eng.run_step([StepEntry(f"q{i}", s[half:], [len(s) - half - 1])]).clone() if len(s) > half else None)
    torch.cuda.synchronize()
    for i, s in enumerate(seqs):
        if outs[i] is None:
            continue
        want = plain.forward(cfg, w, s)[-1]
        err = float((outs[i][0].cpu().double() - want).abs().max() / want.abs().max())
        assert err <= TOL[dtype], f"request {i}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_steps_follow_changes_of_the_batch(folders, dtype):
    """A captured decode step keeps a host copy of its metadata and rewrites
    only what changed.  Here the batch of a captured shape changes under it: a
    request ends and another takes its row, one is ended and begun again under
    the same name, and the order of the rows changes."""
    from inferflux_b200 import StepEntry
    folder, cfg, w = folders["D"]
    seqs = {k: random_tokens(cfg["vocab_size"], 60, 130 + i) for i, k in enumerate("abcd")}
    refs = {k: plain.forward(cfg, w, s).numpy() for k, s in seqs.items()}
    eng = _engine(folder, dtype)
    pos = {}

    def prompt(k, n):
        eng.run_step([StepEntry(k, seqs[k][:n], [])])
        pos[k] = n

    def decode(keys):
        logits = eng.run_step([StepEntry(k, [seqs[k][pos[k]]], [0]) for k in keys]).cpu().numpy()
        for i, k in enumerate(keys):
            err = np.abs(logits[i].astype(np.float64) - refs[k][pos[k]]).max() / np.abs(refs[k]).max()
            assert err <= TOL[dtype], f"request {k} at {pos[k]}: {err:.3e}"
            pos[k] += 1

    for k, n in (("a", 5), ("b", 17), ("c", 30)):
        prompt(k, n)
    for _ in range(7):
        decode("abc")
    replays = eng.runner.graph_replays
    assert replays >= 3
    eng.end_request("b")
    prompt("d", 9)
    for _ in range(3):
        decode("adc")                    # d sits in b's row
    eng.end_request("a")
    prompt("a", 21)                      # the same name, other pages and another length
    for _ in range(3):
        decode("adc")
    for _ in range(3):
        decode("cad")                    # rows in another order
    assert eng.runner.graph_replays >= replays + 9


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_ahead_gives_the_same_tokens(folders, dtype):
    """Decode steps are started before the host has read the ids of the step
    before them.  The tokens are the same as when every step waits for its ids;
    a request that ends on a stop token is found out one step late, and the token
    that step made for it is dropped; a request that reaches its token limit is
    never run past it."""
    from inferflux_b200 import SamplingParams
    folder, cfg, w = folders["A"]
    prompts = [random_tokens(cfg["vocab_size"], n, 140 + n) for n in (6, 19, 11, 30)]
    plain_run = _engine(folder, dtype, pipeline_decode=False)
    greedy = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    base = plain_run.generate(prompts, greedy)
    assert plain_run.stats.get("steps_run_ahead", 0) == 0
    # request 1 stops on the token it would produce 10th, request 2 after 17 tokens, request 3 samples with a seed
    params = [greedy,
              SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True, stop_token_ids=[base[1].tokens[9]]),
              SamplingParams(temperature=0.0, max_tokens=17, ignore_eos=True),
              SamplingParams(temperature=0.9, top_p=0.9, seed=5, max_tokens=40, ignore_eos=True)]
    want = _engine(folder, dtype, pipeline_decode=False).generate(prompts, params)
    ahead = _engine(folder, dtype)
    got = ahead.generate(prompts, params)
    assert ahead.stats["steps_run_ahead"] > 10
    for a, b in zip(want, got):
        assert a.tokens == b.tokens and a.finish_reason == b.finish_reason
    stop_at = base[1].tokens.index(base[1].tokens[9]) + 1
    assert got[1].finish_reason == "stop" and len(got[1].tokens) == stop_at
    assert got[2].finish_reason == "length" and len(got[2].tokens) == 17
    assert ahead.stats["pages_free"] == ahead.stats["pages_total"]


def test_random_arrivals_preemption_and_running_ahead(folders):
    """Thirty requests arrive at random steps into a pool that is too small for
    them (so the youngest give way and start over), some stop on a stop token,
    some at their token limit, some sample with a seed.  In float32 a request's
    tokens do not depend on its company, so every request must come out as when
    it runs alone in a roomy engine that waits for every step's ids."""
    import random
    from inferflux_b200 import SamplingParams
    folder, cfg, w = folders["E"]
    rng = random.Random(7)
    n = 30
    prompts = [random_tokens(cfg["vocab_size"], rng.randint(1, 90), 300 + i) for i in range(n)]
    params = []
    for i in range(n):
        kind = i % 3
        if kind == 0:
            params.append(SamplingParams(temperature=0.0, max_tokens=rng.randint(1, 40), ignore_eos=True))
        elif kind == 1:
            params.append(SamplingParams(temperature=0.7, top_k=20, seed=100 + i, max_tokens=rng.randint(5, 40), ignore_eos=True))
        else:
            params.append(SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True,
                                         stop_token_ids=[rng.randrange(cfg["vocab_size"]) for _ in range(60)]))
    alone = []
    for p, sp in zip(prompts, params):
        alone.append(_engine(folder, "float32", pipeline_decode=False).generate([p], sp)[0])
    eng = _engine(folder, "float32", kv_cache_tokens=400, max_seqs=6, chunked_prefill_tokens=24, max_batch_tokens=64)
    arrive = sorted(rng.randint(0, 60) for _ in range(n))
    done, step, nxt = {}, 0, 0
    while nxt < n or eng.has_work():
        while nxt < n and arrive[nxt] <= step:
            eng.add_request(prompts[nxt], params[nxt], rid=nxt)
            nxt += 1
        for r in eng.step():
            done[r.rid] = r
        step += 1
        assert step < 5000
    assert len(done) == n
    st = eng.stats
    assert st["preemptions"] > 0 and st.get("steps_run_ahead", 0) > 0
    for i in range(n):
        assert done[i].tokens == alone[i].tokens and done[i].finish_reason == alone[i].finish_reason, i
    assert st["pages_free"] == st["pages_total"]
    eng.runner.kv.check(), eng.runner.slots.check()


def test_decoding_with_contexts_of_very_different_lengths(monkeypatch):
    """One request with 1,150 tokens of context beside three short ones: attention for the single tokens
    shares the tiles of all four out evenly over its blocks (the other kernel would make the long context
    wait alone), in eager steps and in captured ones; the logits are the plain implementation's."""
    from inferflux_b200 import StepEntry
    from inferflux_b200.kernels import ops
    cfg = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=96, num_hidden_layers=2,
               num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=160, vocab_size=500,
               rope_theta=300000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=1536,
               use_sliding_window=False, hidden_act="silu", torch_dtype="bfloat16")
    folder = make_model_folder(cfg, seed=91, sharpen=4.0)
    _, cfg, w = (folder, *plain.load_folder(folder))
    calls = {"even": 0, "split": 0}
    even, split, prep = ops.attn_decode_even_bf16, ops.attn_decode_bf16, ops.attn_decode_prep_bf16
    monkeypatch.setattr(ops, "attn_decode_even_bf16", lambda *a, **k: (calls.__setitem__("even", calls["even"] + 1), even(*a, **k))[1])
    monkeypatch.setattr(ops, "attn_decode_bf16", lambda *a, **k: (calls.__setitem__("split", calls["split"] + 1), split(*a, **k))[1])
    monkeypatch.setattr(ops, "attn_decode_prep_bf16", lambda *a, **k: (calls.__setitem__("split", calls["split"] + 1), prep(*a, **k))[1])
    steps = 12
    lengths = [1150, 30, 75, 12]
    seqs = [random_tokens(cfg["vocab_size"], n + steps, 300 + i) for i, n in enumerate(lengths)]
    refs = [plain.forward(cfg, w, s).numpy() for s in seqs]
    eng = _engine(folder, "bfloat16", kv_cache_tokens=2048, max_model_len=1536)
    for i, (s, n) in enumerate(zip(seqs, lengths)):
        for a in range(0, n, 512):
            eng.run_step([StepEntry(f"r{i}", s[a:min(n, a + 512)], [])])
    worst = 0.0
    for p in range(steps):
        logits = eng.run_step([StepEntry(f"r{i}", [s[n + p]], [0]) for i, (s, n) in enumerate(zip(seqs, lengths))]).cpu().numpy()
        for i, n in enumerate(lengths):
            ref = refs[i][n + p]
            worst = max(worst, float(np.abs(logits[i].astype(np.float64) - ref).max() / np.abs(ref).max()))
    assert worst <= TOL["bfloat16"], f"{worst:.3e}"
    assert calls["even"] > 0 and calls["split"] == 0, calls          # layers x (eager steps + the capture)
    assert eng.runner.graph_replays >= steps - 4
    ops.check_device_errors("cuda:0")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_penalties_from_the_device_run_ahead_and_survive_preemption(folders, dtype):
    """Requests with repetition, frequency and presence penalties keep their recent tokens in rings on the
    device, so their decode steps are started ahead like any others; the tokens are those of the engine that
    waits for every step and counts on the host, also when pages run out and a request gives way and starts
    again, and for a window longer than the rings (counted on the host, beside ring-served requests)."""
    from inferflux_b200 import SamplingParams
    folder, cfg, w = folders["A"]
    prompts = [random_tokens(cfg["vocab_size"], n, 170 + n) for n in (9, 21, 14, 33)]
    params = [SamplingParams(temperature=0.0, max_tokens=60, repetition_penalty=1.4, ignore_eos=True),
              SamplingParams(temperature=0.0, max_tokens=60, frequency_penalty=0.8, presence_penalty=0.4, penalty_last_n=10,
                             ignore_eos=True),
              SamplingParams(temperature=0.9, seed=3, max_tokens=60, repetition_penalty=1.2, presence_penalty=0.5,
                             ignore_eos=True),
              SamplingParams(temperature=0.0, max_tokens=60, ignore_eos=True)]
    # the first token of request 0 under its penalty, by the plain implementation
    want0 = plain.apply_penalties(plain.forward(cfg, w, prompts[0])[-1], prompts[0][-64:], 1.4, 0.0, 0.0)
    waiting = _engine(folder, dtype, pipeline_decode=False)
    waiting.sampler.max_seqs = 0                            # no rings: every window is counted on the host
    want = waiting.generate(prompts, params)
    assert waiting.stats.get("steps_run_ahead", 0) == 0
    if dtype == "float32":
        assert want[0].tokens[0] == int(torch.argmax(want0))
    ahead = _engine(folder, dtype)
    got = ahead.generate(prompts, params)
    assert ahead.stats["steps_run_ahead"] > 20
    for a, b in zip(want, got):
        assert a.tokens == b.tokens
    # few pages: requests give way and start again, their rings are seeded again
    tight = _engine(folder, dtype, kv_cache_tokens=192)
    got = tight.generate(prompts, params)
    assert tight.stats["preemptions"] > 0
    for a, b, p, sp in zip(want, got, prompts, params):
        _same_tokens(cfg, w, p, sp, a.tokens, b.tokens, dtype)
    # a window beyond the rings beside one within them
    long_window = [SamplingParams(temperature=0.0, max_tokens=30, repetition_penalty=1.3, penalty_last_n=1000, ignore_eos=True),
                   params[1]]
    a = _engine(folder, dtype, pipeline_decode=False)
    a.sampler.max_seqs = 0
    b = _engine(folder, dtype)
    for x, y in zip(a.generate(prompts[:2], long_window), b.generate(prompts[:2], long_window)):
        assert x.tokens == y.tokens


@pytest.mark.parametrize("pipeline", [True, False])
def test_a_failed_step_hands_out_no_tokens(folders, pipeline):
    """When a kernel's bounded wait runs out it sets the device's error word.
    The engine reads the word before it returns finished requests, whether the
    call that finds them ran ahead of the host or not.  The word is set here by
    hand; no kernel is made to fail."""
    from inferflux_b200 import SamplingParams
    from inferflux_b200.kernels import ops
    folder, cfg, w = folders["A"]
    prompts = [random_tokens(cfg["vocab_size"], 9, 500 + i) for i in range(2)]
    drawn = dict(temperature=1.5, seed=5, max_tokens=30)                 # in float32 the draws do not depend on the batch
    first = _engine(folder, "float32").generate(prompts[:1], SamplingParams(ignore_eos=True, **drawn))[0].tokens
    k = next(i for i in range(5, 30) if first[i] not in first[:i])       # stops at its k-th token, on a stop token:
    eng = _engine(folder, "float32", pipeline_decode=pipeline)           # found out one step late when running ahead
    eng.add_request(prompts[0], SamplingParams(stop_token_ids=[first[k]], **drawn))
    eng.add_request(prompts[1], SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True))
    for _ in range(4):
        assert eng.step() == []
    if pipeline:
        assert eng.stats["steps_run_ahead"] > 0
    ops.error_flag(eng.engine_config.device).fill_(1)
    with pytest.raises(ops.KernelError):
        for _ in range(k + 2):
            eng.step()
    assert int(ops.error_flag(eng.engine_config.device).item()) == 0     # read and cleared
