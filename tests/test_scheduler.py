"""The scheduler's decisions (host logic over a fake cache, no GPU): admission,
portions under the token budget, decode first, finishing and freeing, and
what happens when pages run out."""
from __future__ import annotations

import random

import pytest

from inferflux_b200.cache import KVCacheManager, StateSlotManager
from inferflux_b200.config import EngineConfig
from inferflux_b200.engine.scheduler import CacheView, Phase, Request, Scheduler
from inferflux_b200.parts.base import KVNeed
from inferflux_b200.sampling import SamplingParams


class FakeCache(CacheView):
    """The real page and slot bookkeeping without any device memory."""

    def __init__(self, pages, page_size=16, max_seqs=8, needs=None):
        self.kv = KVCacheManager(needs or [KVNeed.keys_and_values(1, 16)], pages, page_size)
        self.slots = StateSlotManager(max_seqs)

    def pages_needed(self, rid, n_new):
        return self.kv.pages_needed(rid, n_new, 0)

    def free_pages(self):
        return [p.num_free for p in self.kv.pools]

    def total_pages(self):
        return [p.num_pages for p in self.kv.pools]

    def free_slots(self):
        return self.slots.num_free

    def has(self, rid):
        return self.kv.has(rid)

    def release(self, rid):
        self.kv.free_request(rid)
        self.slots.release(rid)

    @property
    def page_size(self):
        return self.kv.page_size

    def run(self, plan):
        """What the step function does to the cache."""
        for it in plan.items:
            rid = it.request.rid
            if not self.kv.has(rid):
                self.kv.add_request(rid)
                self.slots.acquire(rid)
            assert self.kv.length(rid) == it.start
            self.kv.reserve(rid, it.count)
        for it in plan.items:
            self.kv.advance(it.request.rid, it.count)
        self.kv.check()
        self.slots.check()


def make(pages=(64,), **kw):
    opts = dict(max_batch_tokens=64, max_batch_size=8, chunked_prefill_tokens=32, max_seqs=8, page_size=16)
    opts.update(kw)
    cache = FakeCache(list(pages), opts["page_size"], opts["max_seqs"])
    return Scheduler(EngineConfig(**opts), cache, max_model_len=4096), cache


def req(rid, n_prompt, max_tokens=4, **kw):
    return Request(rid=rid, prompt=list(range(1, n_prompt + 1)),
                   params=SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True, **kw))


def drive(s, cache, token=7, limit=10000):
    """Run plans to completion with a constant sampled token; returns the plans."""
    plans = []
    while s.has_work():
        plan = s.schedule()
        s.begin_step(plan)
        cache.run(plan)
        s.finish_step(plan, {it.request.rid: token for it in plan.items if it.samples})
        plans.append(plan)
        assert len(plans) < limit, "the scheduler does not finish"
    return plans


def test_prompt_is_cut_into_portions_under_the_cap():
    s, cache = make(chunked_prefill_tokens=32, max_batch_tokens=1000)
    r = req("a", 100)
    s.add(r)
    plans = drive(s, cache)
    counts = [[(it.count, it.samples) for it in p.items] for p in plans]
    assert counts[:4] == [[(32, False)], [(32, False)], [(32, False)], [(4, True)]]      # logits only at the end
    assert all(c == [(1, True)] for c in counts[4:]) and len(counts) == 4 + 3
    assert r.phase is Phase.FINISHED and r.finish_reason == "length" and r.output == [7] * 4
    assert cache.free_pages() == [64] and cache.free_slots() == 8                       # freed at the end


def test_decodes_first_then_prompts_share_the_budget():
    s, cache = make(max_batch_tokens=40, chunked_prefill_tokens=32)
    a, b, c = req("a", 8, 50), req("b", 60, 5), req("c", 60, 5)
    s.add(a)
    plan = s.schedule(); s.begin_step(plan); cache.run(plan); s.finish_step(plan, {"a": 1})
    s.add(b); s.add(c)
    plan = s.schedule()
    got = [(it.request.rid, it.count) for it in plan.items]
    # a decodes (1 token); the other 39 tokens go to b (cap 32) and then c (7 left)
    assert got == [("a", 1), ("b", 32), ("c", 7)]
    assert plan.n_tokens == 40


def test_mixed_prefill_budget_ratio_limits_prompts():
    s, cache = make(max_batch_tokens=40, chunked_prefill_tokens=32, mixed_prefill_budget_ratio=0.5)
    s.add(req("a", 100))
    plan = s.schedule()
    assert [(it.count) for it in plan.items] == [20]


def test_max_batch_size_and_slots_limit_admission():
    s, cache = make(max_batch_size=2, max_batch_tokens=1000)
    for i in range(4):
        s.add(req(f"r{i}", 5))
    plan = s.schedule()
    assert [it.request.rid for it in plan.items] == ["r0", "r1"]
    s2, cache2 = make(max_seqs=1, max_batch_tokens=1000)
    for i in range(2):
        s2.add(req(f"r{i}", 5))
    assert [it.request.rid for it in s2.schedule().items] == ["r0"]       # one state slot: one request
    plans = drive(s2, cache2)
    assert all(len(p.items) == 1 for p in plans)


def test_arrival_order_is_kept_when_pages_are_short():
    s, cache = make(pages=(4,), max_batch_tokens=1000, chunked_prefill_tokens=1000)
    s.add(req("big", 60, 2))          # 4 pages: takes the whole pool
    s.add(req("small", 3, 2))
    plan = s.schedule()
    assert [(it.request.rid, it.count) for it in plan.items] == [("big", 60)]   # small does not jump the queue
    plans = drive(s, cache)
    assert s.stats["finished"] == 2 and cache.free_pages() == [4]


def test_portion_is_cut_to_the_pages_that_are_free():
    s, cache = make(pages=(5,), max_batch_tokens=1000, chunked_prefill_tokens=1000)
    a = req("a", 40, 30)
    s.add(a)
    plan = s.schedule(); s.begin_step(plan); cache.run(plan); s.finish_step(plan, {"a": 1})   # a holds 3 pages
    s.add(req("b", 70, 2))
    plan = s.schedule()
    got = {it.request.rid: it.count for it in plan.items}
    assert got == {"a": 1, "b": 32}                                       # 2 free pages = 32 tokens of b


def test_out_of_pages_preempts_the_youngest_and_recomputes():
    s, cache = make(pages=(4,), max_batch_tokens=1000, chunked_prefill_tokens=1000)
    old, young = req("old", 30, 30), req("young", 30, 30)
    s.add(old); s.add(young)
    plans = drive(s, cache)
    assert young.preemptions >= 1 and old.preemptions == 0               # the older request never gives way
    assert old.finish_reason == "length" and young.finish_reason == "length"
    assert len(old.output) == 30 and len(young.output) == 30             # nothing sampled twice, nothing lost
    assert s.stats["preemptions"] == young.preemptions
    # after giving way the request was recomputed from prompt + output so far
    recomputed = [it for p in plans for it in p.items if it.request is young and it.start == 0]
    assert len(recomputed) == 1 + young.preemptions
    assert cache.free_pages() == [4] and cache.free_slots() == 8


def test_request_larger_than_the_pool():
    s, cache = make(pages=(4,))
    big = req("big", 64, 4)           # prompt + 1 token needs 5 pages
    s.add(big)
    assert big.phase is Phase.FINISHED and big.finish_reason == "prompt_too_long" and not s.has_work()
    grows = req("grows", 60, 100)     # fits at first, outgrows the pool while decoding alone
    s.add(grows)
    drive(s, cache)
    assert grows.finish_reason == "cache_full" and len(grows.output) == 5   # 64 tokens cached = the pool; the 5th sampled token has no page
    assert cache.free_pages() == [4]


def test_stop_tokens_and_eos():
    s, cache = make()
    a = Request("a", [1, 2, 3], SamplingParams(temperature=0.0, max_tokens=50), eos_token_id=7)
    b = Request("b", [1, 2, 3], SamplingParams(temperature=0.0, max_tokens=50, stop_token_ids=[7]))
    c = Request("c", [1, 2, 3], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True), eos_token_id=7)
    for r in (a, b, c):
        s.add(r)
    drive(s, cache, token=7)
    assert (a.finish_reason, a.output) == ("stop", [7]) and (b.finish_reason, b.output) == ("stop", [7])
    assert (c.finish_reason, c.output) == ("length", [7, 7, 7])


def test_random_workloads_finish_and_free_everything():
    rng = random.Random(3)
    for trial in range(25):
        pages = rng.randint(6, 30)
        s, cache = make(pages=(pages,), max_batch_tokens=rng.choice([16, 48, 200]),
                        chunked_prefill_tokens=rng.choice([8, 32, 100]), max_batch_size=rng.choice([2, 4, 8]),
                        max_seqs=rng.choice([2, 4, 8]))
        reqs = [req(f"r{i}", rng.randint(1, 70), rng.randint(1, 30)) for i in range(rng.randint(1, 12))]
        for r in reqs:
            s.add(r)
        plans = drive(s, cache)
        for p in plans:
            assert p.n_tokens <= s.cfg.max_batch_tokens and len(p.items) <= s.cfg.max_batch_size
            assert len({it.request.rid for it in p.items}) == len(p.items)
        for r in reqs:
            assert r.phase is Phase.FINISHED
            if r.finish_reason == "length":
                assert len(r.output) == r.params.max_tokens
            else:
                assert r.finish_reason in ("cache_full", "prompt_too_long")
        assert cache.free_pages() == [pages] and cache.free_slots() == s.cfg.max_seqs


def test_token_slice_equals_the_slice_of_all_tokens():
    from inferflux_b200.engine.scheduler import Request
    from inferflux_b200.sampling.params import SamplingParams
    r = Request(rid="x", prompt=[1, 2, 3, 4, 5], params=SamplingParams(), output=[6, 7, 8])
    for start in range(0, 8):
        for count in range(1, 9 - start):
            assert r.token_slice(start, count) == r.tokens[start:start + count]


def test_contexts_skewed_rule():
    """Which steps of single tokens count as having contexts of very different lengths."""
    from inferflux_b200.parts.attention import contexts_skewed
    assert not contexts_skewed([4096] * 8)                     # equal
    assert not contexts_skewed([4096])                         # one request
    assert not contexts_skewed([900, 10, 10, 10])              # nothing long
    assert contexts_skewed([32768] + [1024] * 63)
    assert contexts_skewed([1150, 30, 75, 12])
    assert not contexts_skewed([2048, 1800, 1500, 1900])       # longest below 1.5 times the mean


def test_a_step_that_fails_gives_back_what_it_seated(tmp_path):
    """The step function seats new requests and holds pages before it runs.
    When the run raises (here: on the CPU every kernel refuses), requests
    seated by that call are ended again; one known before keeps its place."""
    import torch
    from helpers import TINY_A, make_model_folder
    from inferflux_b200.config import EngineConfig, build_spec, load_config
    from inferflux_b200.engine import Model, StepEntry, StepRunner
    from inferflux_b200.kernels.ops import KernelError
    folder = make_model_folder(TINY_A, 0, str(tmp_path / "m"))
    model = Model(build_spec(load_config(folder)), torch.float32, "cpu")
    model.load_folder(folder)
    runner = StepRunner(model, EngineConfig(dtype="float32", device="cpu", kv_cache_tokens=256, max_seqs=2))
    free = runner.kv.num_free(0)
    with pytest.raises(KernelError):
        runner.step([StepEntry("a", [1, 2, 3], [2])])
    assert not runner.has("a") and runner.slots.num_free == 2 and runner.kv.num_free(0) == free
    runner.begin("known")
    with pytest.raises(KernelError):
        runner.step([StepEntry("known", list(range(20)), []), StepEntry("new", [4], [0])])
    assert runner.has("known") and not runner.has("new") and runner.slots.num_free == 1
    assert runner.length("known") == 0 and runner.kv.num_free(0) == free - 2     # 20 tokens: two pages stay held
    runner.end("known")
    assert runner.kv.num_free(0) == free and runner.slots.num_free == 2
    runner.kv.check()
