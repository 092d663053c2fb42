"""The scheduler: which requests run in the next step, and with how many tokens.

Every step the batch is formed anew (iteration-level scheduling):

1. Requests that are decoding get one token each, oldest first, up to
   ``max_batch_size`` requests.
2. The rest of the token budget goes to prompts, first those already begun,
   then waiting ones in arrival order.  The budget for prompts is
   ``floor(max_batch_tokens * mixed_prefill_budget_ratio)`` minus the decode
   tokens, at least 1; one request gets at most ``chunked_prefill_tokens`` per
   step (the reference's chunk cap and budget rule,
   runtime/execution/batch_executor.cpp:196-213, scheduler/scheduler.h:74-84).
3. A waiting request is admitted only if a state slot is free and the pools
   can hold its next portion (the reference needs a sequence lease and
   ``ceil(prompt/16) + 1`` blocks, scheduler/scheduler.cpp:1827-1877).

When pages run out:

* a prompt portion is cut down to the tokens that still fit; if none fit, the
  request waits (nothing is admitted past it: arrival order is kept);
* a decoding request that cannot get the page for its next token makes the
  *youngest* running request give way: its pages and slot are given back and it
  returns to the head of the waiting queue, to be recomputed from its prompt
  plus the tokens it has produced (their sampling is not repeated);
* a request that cannot run even alone (it needs more pages than the pool has)
  is finished with reason ``cache_full`` (at admission: ``prompt_too_long``).

The reference instead swaps bookkeeping to a host pool or falls back to a
single-sequence path (scheduler/scheduler.cpp:1843-1877,2064-2077).

The scheduler is host-only logic over a small interface to the cache
(:class:`CacheView`), so its decisions are tested without a GPU.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams


class CacheView:
    """What the scheduler needs to know of the cache (StepRunner provides it)."""

    def pages_needed(self, rid: Optional[Hashable], n_new: int) -> List[int]:
        raise NotImplementedError

    def free_pages(self) -> List[int]:
        raise NotImplementedError

    def total_pages(self) -> List[int]:
        raise NotImplementedError

    def free_slots(self) -> int:
        raise NotImplementedError

    def has(self, rid: Hashable) -> bool:
        raise NotImplementedError

    def release(self, rid: Hashable) -> None:
        raise NotImplementedError

    @property
    def page_size(self) -> int:
        raise NotImplementedError


class Phase(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass
class Request:
    rid: Hashable
    prompt: List[int]
    params: SamplingParams
    eos_token_id: Optional[int] = None
    arrival: int = 0
    seed: int = 0
    phase: Phase = Phase.WAITING
    output: List[int] = field(default_factory=list)
    computed: int = 0                 # tokens whose keys and values are in the cache
    finish_reason: Optional[str] = None
    preemptions: int = 0

    @property
    def tokens(self) -> List[int]:
        """Everything the cache must hold before the next token can be sampled."""
        return self.prompt + self.output

    def token_slice(self, start: int, count: int) -> List[int]:
        """``tokens[start:start + count]`` without joining the two lists."""
        n = len(self.prompt)
        if start >= n:
            return self.output[start - n:start - n + count]
        if start + count <= n:
            return self.prompt[start:start + count]
        return self.prompt[start:] + self.output[:start + count - n]

    @property
    def remaining(self) -> int:
        return len(self.prompt) + len(self.output) - self.computed

    @property
    def decoding(self) -> bool:
        return self.phase is Phase.RUNNING and self.remaining == 1 and len(self.output) > 0


@dataclass
class Planned:
    request: Request
    start: int            # first token (index into request.tokens) of this portion
    count: int
    samples: bool         # the portion ends the known tokens: its last logits give the next token


@dataclass
class StepPlan:
    items: List[Planned] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    finished: List[Request] = field(default_factory=list)   # finished by the scheduler itself (cache_full ...)

    @property
    def n_tokens(self) -> int:
        return sum(p.count for p in self.items)


class Scheduler:
    def __init__(self, cfg: EngineConfig, cache: CacheView, max_model_len: int):
        cfg.validate()
        self.cfg = cfg
        self.cache = cache
        self.max_model_len = max_model_len
        self.waiting: List[Request] = []
        self.running: List[Request] = []
        self._arrivals = 0
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0,
                      "finished": 0, "rejected": 0}

    # -------------------------------------------------------------- intake
    def add(self, request: Request) -> None:
        request.params.validate()
        if not request.prompt:
            raise ValueError(f"request {request.rid!r}: empty prompt")
        request.arrival = self._arrivals
        self._arrivals += 1
        request.phase = Phase.WAITING
        ps = self.cache.page_size
        # the prompt plus one sampled token must fit the pools and the model length
        need = (len(request.prompt) + 1 + ps - 1) // ps
        if len(request.prompt) + 1 > self.max_model_len or any(need > t for t in self.cache.total_pages()):
            self._finish(request, "prompt_too_long")
            self.stats["rejected"] += 1
            return
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------ planning
    def schedule(self) -> StepPlan:
        plan = StepPlan()
        cfg = self.cfg
        state = {"free": list(self.cache.free_pages()), "slots": self.cache.free_slots()}

        def refresh() -> None:
            """Free pages after an eviction, less what this plan has promised."""
            free = list(self.cache.free_pages())
            for it in plan.items:
                new = it.request.phase is Phase.WAITING
                for g, k in enumerate(self._need(it.request, it.count, new)):
                    free[g] -= k
            state["free"] = free
            state["slots"] = self.cache.free_slots() - sum(
                1 for it in plan.items if it.request.phase is Phase.WAITING)

        def make_room(req: Request, n: int, protected: List[Request]) -> bool:
            """Evict the youngest running requests (never ``req`` or the
            protected ones) until ``n`` tokens of ``req`` fit."""
            while not self._fits(req, n, state["free"], False):
                victim = self._youngest_running(exclude=protected + [req])
                if victim is None:
                    return False
                self._preempt(victim, plan)
                refresh()
            return True

        def promise(req: Request, n: int, new: bool) -> None:
            for g, k in enumerate(self._need(req, n, new)):
                state["free"][g] -= k
            if new:
                state["slots"] -= 1

        # 1. one token for every decoding request, oldest first
        scheduled: List[Request] = []
        for req in sorted((r for r in self.running if r.decoding), key=lambda r: r.arrival):
            if req.phase is not Phase.RUNNING:
                continue                       # gave way to an older request a moment ago
            if len(plan.items) >= cfg.max_batch_size or plan.n_tokens >= cfg.max_batch_tokens:
                break
            if not make_room(req, 1, scheduled):
                if scheduled or len(self.running) > 1:
                    self._preempt(req, plan)   # the youngest left: it gives way itself
                    refresh()
                else:                          # alone with the whole pool and still no page
                    self._release(req)
                    self._finish(req, "cache_full")
                    plan.finished.append(req)
                    refresh()
                continue
            promise(req, 1, False)
            plan.items.append(Planned(req, req.computed, 1, True))
            scheduled.append(req)

        # 2. prompt portions: begun ones first, then waiting ones in arrival order
        n_decode = plan.n_tokens
        budget = max(1, int(cfg.max_batch_tokens * cfg.mixed_prefill_budget_ratio) - n_decode)
        budget = min(budget, cfg.max_batch_tokens - n_decode)
        begun = sorted((r for r in self.running if not r.decoding and r.remaining > 0), key=lambda r: r.arrival)
        for req in begun:
            if budget <= 0 or len(plan.items) >= cfg.max_batch_size:
                break
            if req.phase is not Phase.RUNNING:
                continue
            n = min(req.remaining, cfg.chunked_prefill_tokens, budget)
            n = self._largest_fit(req, n, state["free"], False)
            if n <= 0:
                # an older prompt must not starve behind younger ones that hold the pages
                if not make_room(req, 1, scheduled):
                    continue
                n = self._largest_fit(req, min(req.remaining, cfg.chunked_prefill_tokens, budget),
                                      state["free"], False)
                if n <= 0:
                    continue
            promise(req, n, False)
            plan.items.append(Planned(req, req.computed, n, n == req.remaining))
            scheduled.append(req)
            budget -= n
        for req in list(self.waiting):
            if budget <= 0 or len(plan.items) >= cfg.max_batch_size or state["slots"] <= 0:
                break
            if req in plan.preempted:
                break                          # it gave way in this very step: no room for it yet
            n = min(req.remaining, cfg.chunked_prefill_tokens, budget)
            n = self._largest_fit(req, n, state["free"], True)
            if n <= 0:
                break                          # keep arrival order: nobody jumps the queue
            promise(req, n, True)
            plan.items.append(Planned(req, req.computed, n, n == req.remaining))
            budget -= n
        # nothing can move: the oldest request needs more than the pool holds
        if not plan.items and not plan.finished and not plan.preempted and self.has_work():
            stuck = min(self.running + self.waiting, key=lambda r: r.arrival)
            if stuck.phase is Phase.RUNNING:
                self._release(stuck)
            else:
                self.waiting.remove(stuck)
            self._finish(stuck, "cache_full")
            plan.finished.append(stuck)
        return plan

    def _need(self, req: Request, n: int, new: bool) -> List[int]:
        if new:
            # a waiting request has nothing in the cache (after giving way it starts over)
            return self.cache.pages_needed(None, n)
        return self.cache.pages_needed(req.rid, n)

    def _fits(self, req: Request, n: int, free: Sequence[int], new: bool) -> bool:
        return all(k <= f for k, f in zip(self._need(req, n, new), free))

    def _largest_fit(self, req: Request, n: int, free: Sequence[int], new: bool) -> int:
        lo, hi = 0, n
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if self._fits(req, mid, free, new):
                lo = mid
            else:
                hi = mid - 1
        return lo

    def _youngest_running(self, exclude: Sequence[Request]) -> Optional[Request]:
        cands = [r for r in self.running if r not in exclude]
        return max(cands, key=lambda r: r.arrival) if cands else None

    def _release(self, req: Request) -> None:
        if self.cache.has(req.rid):
            self.cache.release(req.rid)
        if req in self.running:
            self.running.remove(req)

    def _preempt(self, req: Request, plan: StepPlan) -> None:
        self._release(req)
        req.phase = Phase.WAITING
        req.computed = 0
        req.preemptions += 1
        self.stats["preemptions"] += 1
        # back to the head of the queue, before younger waiting requests
        idx = 0
        while idx < len(self.waiting) and self.waiting[idx].arrival < req.arrival:
            idx += 1
        self.waiting.insert(idx, req)
        plan.preempted.append(req)
        plan.items = [it for it in plan.items if it.request is not req]

    def _finish(self, req: Request, reason: str) -> None:
        req.phase = Phase.FINISHED
        req.finish_reason = reason
        self.stats["finished"] += 1

    # ------------------------------------------------------------- results
    def begin_step(self, plan: StepPlan) -> None:
        """Move the plan's waiting requests to running (call before the step runs)."""
        for it in plan.items:
            req = it.request
            if req.phase is Phase.WAITING:
                self.waiting.remove(req)
                self.running.append(req)
                req.phase = Phase.RUNNING

    def finish_step(self, plan: StepPlan, sampled: Dict[Hashable, int]) -> List[Request]:
        """Record the step: advance what was computed, append sampled tokens,
        finish and free requests that are done.  Returns those finished now."""
        done: List[Request] = []
        self.stats["steps"] += 1
        for it in plan.items:
            req = it.request
            req.computed += it.count
            if it.count == 1 and req.output:
                self.stats["decode_tokens"] += 1
            else:
                self.stats["prefill_tokens"] += it.count
            if not it.samples:
                continue
            tok = int(sampled[req.rid])
            req.output.append(tok)
            p = req.params
            reason = None
            if not p.ignore_eos and req.eos_token_id is not None and tok == req.eos_token_id:
                reason = "stop"
            elif tok in p.stop_token_ids:
                reason = "stop"
            elif len(req.output) >= p.max_tokens:
                reason = "length"
            elif len(req.prompt) + len(req.output) >= self.max_model_len:
                reason = "length"
            if reason:
                self._release(req)
                self._finish(req, reason)
                done.append(req)
        return done
