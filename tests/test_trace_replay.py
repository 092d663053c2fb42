"""bin/trace_run against the plain implementation: the same requests replayed
whole, with the last 32 tokens one by one, in portions of changing size, and
mixed with other requests in a pool so small that pages are used again; in
float32 and in bfloat16; for tiny configurations that differ in every size."""
from __future__ import annotations

import random

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from helpers import TINY, TOL, TraceProcess, make_model_folder, random_tokens, rel_err

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [70, 33, 5, 130, 64, 97], "B": [70, 40, 9, 150, 65, 111, 1], "C": [50, 81, 17, 100],
           "D": [150, 66, 3, 129, 90], "E": [70, 40, 9, 150, 65, 111, 1]}


def max_live_tokens(lengths) -> int:
    """What --max-tokens promises to hold: the four longest requests, each
    rounded up to a multiple of 64.  All requests together, replayed twice in
    the mixed test, are more than that, so pages must be used again."""
    return sum((n + 63) // 64 * 64 for n in sorted(lengths)[-4:])


class Case:
    def __init__(self, name: str, dtype: str):
        cfg = TINY[name]
        self.name, self.dtype = name, dtype
        self.folder = make_model_folder(cfg, seed=ord(name), sharpen=4.0,
                                        vector_dtype=torch.float32 if name in "BE" else None)
        self.cfg, self.weights = plain.load_folder(self.folder)
        self.requests = [random_tokens(cfg["vocab_size"], n, 100 + i) for i, n in enumerate(LENGTHS[name])]
        self.refs = [plain.forward(self.cfg, self.weights, r).numpy() for r in self.requests]
        self.proc = TraceProcess(self.folder, dtype, max_live_tokens(LENGTHS[name]))

    def check(self, rid_index: int, start: int, got: np.ndarray, what: str):
        ref = self.refs[rid_index][start:start + got.shape[0]]
        scale = np.abs(self.refs[rid_index]).max()
        err = np.abs(got.astype(np.float64) - ref).max() / scale
        assert err <= TOL[self.dtype], (f"{self.name}/{self.dtype} {what}: request {rid_index} positions "
                                        f"{start}..{start + got.shape[0] - 1}: error {err:.3e} of scale")
        return err


_cases = {}


@pytest.fixture(params=[(n, d) for n in ("A", "B", "C", "D", "E") for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}", scope="module")
def case(request):
    key = request.param
    if key not in _cases:
        _cases[key] = Case(*key)
    yield _cases[key]


def teardown_module(module):
    for c in _cases.values():
        assert c.proc.close() == 0


def test_whole(case):
    """Each request alone, its whole prompt in one step, logits at every position."""
    for i, toks in enumerate(case.requests):
        got = case.proc.step([dict(id=f"w{i}", tokens=toks, want=list(range(len(toks))))], end=[f"w{i}"])
        case.check(i, 0, got, "whole")


def test_prefix_then_one_by_one(case):
    """All but the last 32 tokens in one step, then the last 32 one by one."""
    for i, toks in enumerate(case.requests):
        rid = f"d{i}"
        head = max(1, len(toks) - 32)
        got = case.proc.step([dict(id=rid, tokens=toks[:head], want=[head - 1])])
        case.check(i, head - 1, got, "prefix")
        for p in range(head, len(toks)):
            got = case.proc.step([dict(id=rid, tokens=[toks[p]], want=[0])],
                                 end=[rid] if p == len(toks) - 1 else [])
            case.check(i, p, got, "one by one")
        if head == len(toks):
            case.proc.step([], end=[rid])


def test_portions_of_changing_size(case):
    """Portions of 2, 3, 17, 1, 16, 5, 32, ... tokens; logits at every position."""
    sizes = [2, 3, 17, 1, 16, 5, 32, 2, 15, 64, 2]
    for i, toks in enumerate(case.requests):
        rid, pos, k = f"p{i}", 0, i
        while pos < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - pos)
            k += 1
            last = pos + n == len(toks)
            got = case.proc.step([dict(id=rid, tokens=toks[pos:pos + n], want=list(range(n)))],
                                 end=[rid] if last else [])
            case.check(i, pos, got, f"portion of {n}")
            pos += n


def test_mixed_with_page_reuse(case):
    """Up to four live requests; portions of some beside single tokens of
    others; requests join as others end, so freed pages are used again."""
    rng = random.Random(7)
    order = list(range(len(case.requests))) * 2          # every request twice: the pool turns over
    before = case.proc.stats()
    assert 2 * sum(LENGTHS[case.name]) > max_live_tokens(LENGTHS[case.name])
    waiting = [(f"m{j}_{i}", i) for j, i in enumerate(order)]
    live = {}                                            # rid -> [request index, position]
    while waiting or live:
        while waiting and len(live) < 4:
            rid, i = waiting.pop(0)
            live[rid] = [i, 0]
        entries, ends, checks = [], [], []
        for rid, (i, pos) in list(live.items()):
            toks = case.requests[i]
            if rng.random() < 0.15 and len(live) > 1:
                continue                                 # this request sits the step out
            left = len(toks) - pos
            n = 1 if left <= 32 else min(left - 32, rng.choice([2, 3, 7, 16, 29, 48]))
            want = list(range(n)) if n <= 3 else sorted(rng.sample(range(n), 3))
            entries.append(dict(id=rid, tokens=toks[pos:pos + n], want=want))
            checks.append((i, pos, want))
            live[rid][1] = pos + n
            if pos + n == len(toks):
                ends.append(rid)
                del live[rid]
        if not entries:
            continue
        got = case.proc.step(entries, end=ends)
        row = 0
        for i, pos, want in checks:
            for w in want:
                case.check(i, pos + w, got[row:row + 1], "mixed")
                row += 1
    after = case.proc.stats()
    handed_out = [a - b for a, b in zip(after["page_allocations"], before["page_allocations"])]
    used_again = [a - b for a, b in zip(after["page_reuses"], before["page_reuses"])]
    # more pages were handed out than the pool has, so some were used a second time during this very test
    assert all(h > t for h, t in zip(handed_out, after["pages_total"])), (handed_out, after)
    assert all(u > 0 for u in used_again), (used_again, after)
    assert after["pages_free"] == after["pages_total"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_weights_without_a_folder(tmp_path, dtype):
    """``--random CONFIG.json --seed S`` is the model that ``inferctl random``
    writes for that configuration and seed: the same logits, bit for bit."""
    import json
    from inferflux_b200.config import load_config
    from inferflux_b200.weights.random_init import write_random_model
    cfg = TINY["C"]
    folder = write_random_model(str(tmp_path / "m"), load_config(dict(cfg)), 5)
    (tmp_path / "c.json").write_text(json.dumps(cfg))
    toks = random_tokens(cfg["vocab_size"], 40, 3)
    step = [dict(id="a", tokens=toks, want=[0, 17, 39])]
    from_folder = TraceProcess(folder, dtype, 64)
    from_seed = TraceProcess(None, dtype, 64, extra=["--random", str(tmp_path / "c.json"), "--seed", "5"])
    a, b = from_folder.step(step, end=["a"]), from_seed.step(step, end=["a"])
    assert from_folder.close() == 0 and from_seed.close() == 0
    assert np.array_equal(a, b)
    ref = plain.forward(*plain.load_folder(folder), toks).numpy()[[0, 17, 39]]
    assert rel_err(a, ref) <= TOL[dtype]
