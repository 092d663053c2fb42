"""The Python entry point: load a model, generate tokens.

    from inferflux_b200 import Engine, SamplingParams
    engine = Engine.from_pretrained("model_dir", dtype="bfloat16")
    outputs = engine.generate([[1, 2, 3], [4, 5]], SamplingParams(temperature=0.0, max_tokens=16))

The engine owns one :class:`StepRunner` (model + cache + step function), one
:class:`Scheduler` and one :class:`Sampler`.  The reference has no Python
entry point; its direct generation loop is ``NativeGpuBackend::Generate``
(runtime/backends/native/native_gpu_backend.cpp:523-745): prefill the prompt,
then one token per step until EOS or ``max_tokens``.  Here the same loop runs
through the scheduler, so several prompts share steps.
"""
from __future__ import annotations

import gc
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..config import EngineConfig, ModelConfig, build_spec, load_config
from ..kernels import ops
from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .model import Model
from .runner import StepRunner, torch_dtype
from ..cache import OutOfPages, OutOfSlots
from .scheduler import CacheView, Phase, Planned, Request, Scheduler, StepPlan


@dataclass
class _Launched:
    """A step that has been started: its plan, the requests it samples for, their
    ids on the device and (once the event has passed) on the host."""
    plan: StepPlan
    sampling: List[Request]
    ids: Optional[torch.Tensor]
    host: Optional[torch.Tensor]
    event: Optional[object]


@dataclass
class GenerationResult:
    rid: Hashable
    prompt_tokens: int
    tokens: List[int]
    finish_reason: str
    preemptions: int = 0


class _RunnerCacheView(CacheView):
    def __init__(self, runner: StepRunner):
        self.runner = runner

    def pages_needed(self, rid, n_new):
        return self.runner.kv.pages_needed(rid, n_new, 0)

    def free_pages(self):
        return [p.num_free for p in self.runner.kv.pools]

    def total_pages(self):
        return [p.num_pages for p in self.runner.kv.pools]

    def free_slots(self):
        return self.runner.slots.num_free

    def has(self, rid):
        return self.runner.has(rid)

    def release(self, rid):
        self.runner.end(rid)

    @property
    def page_size(self):
        return self.runner.page_size


class Engine:
    def __init__(self, model: Model, config: ModelConfig, engine_config: EngineConfig):
        self.model = model
        self.config = config
        self.engine_config = engine_config
        self.runner = StepRunner(model, engine_config)
        self.scheduler = Scheduler(engine_config, _RunnerCacheView(self.runner), self.runner.max_model_len)
        self.sampler = Sampler(model.spec.vocab_size, engine_config.device, engine_config.seed, engine_config.max_seqs)
        self._ring_seeded: Dict[Hashable, int] = {}             # request -> its count of preemptions when its ring was seeded
        self._next_id = 0
        self._requests: Dict[Hashable, Request] = {}
        self._inflight: Optional[_Launched] = None              # a started step whose ids the host has not read yet
        pinned = torch.device(engine_config.device).type == "cuda"
        self._id_buffers = [torch.zeros(engine_config.max_batch_size + engine_config.max_seqs, dtype=torch.int32,
                                        pin_memory=pinned) for _ in range(2)]
        self._id_turn = 0

    # ------------------------------------------------------------ construction
    @classmethod
    def from_pretrained(cls, model_dir: str, dtype: str = "bfloat16", **engine_options) -> "Engine":
        """Load ``config.json`` and the safetensors weights of ``model_dir``."""
        ecfg = EngineConfig(dtype=dtype, **engine_options)
        ecfg.validate()
        _require_cuda(ecfg.device)
        config = load_config(model_dir)
        model = Model(build_spec(config), torch_dtype(dtype), ecfg.device)
        model.load_folder(model_dir)
        return cls(model, config, ecfg)

    @classmethod
    def from_config(cls, config: Union[ModelConfig, dict], seed: int = 0, dtype: str = "bfloat16",
                    as_written: bool = False, **engine_options) -> "Engine":
        """A model of ``config``'s architecture with random weights from ``seed``
        (no folder is written).  By default they are drawn on the device, which
        is quick for large models; ``as_written`` draws them on the CPU, the very
        tensors of the folder that ``write_random_model`` writes for the seed."""
        from ..weights.random_init import random_tensors, random_tensors_as_loaded
        ecfg = EngineConfig(dtype=dtype, **engine_options)
        ecfg.validate()
        _require_cuda(ecfg.device)
        if isinstance(config, dict):
            config = load_config(config)
        td = torch_dtype(dtype)
        model = Model(build_spec(config), td, ecfg.device)
        if as_written:
            model.load(random_tensors_as_loaded(model.weight_specs(), seed, td, ecfg.device))
        else:
            model.load(random_tensors(model.weight_specs(), seed, td, torch.float32, ecfg.device))
        return cls(model, config, ecfg)

    # -------------------------------------------------------------- requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    rid: Optional[Hashable] = None) -> Hashable:
        params = params or SamplingParams()
        if rid is None:
            rid = f"req-{self._next_id}"
            self._next_id += 1
        if rid in self._requests and self._requests[rid].phase is not Phase.FINISHED:
            raise KeyError(f"request {rid!r} is still running")
        vocab = self.model.spec.vocab_size
        prompt = [int(t) for t in prompt]
        for t in prompt:
            if not 0 <= t < vocab:
                raise ValueError(f"token id {t} is outside the vocabulary [0, {vocab})")
        seed = params.seed if params.seed is not None else self.sampler.fresh_seed()
        req = Request(rid=rid, prompt=prompt, params=params,
                      eos_token_id=getattr(self.config, "eos_token_id", None), seed=seed)
        self._requests[rid] = req
        self.scheduler.add(req)
        return rid

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    def step(self) -> List[GenerationResult]:
        """Plan one step, run it, sample; returns the requests found finished.

        The ids sampled by a step are read by the host one call later: a call
        first starts the next step and only then waits for the previous step's
        ids, when that next step is known without them (see
        :meth:`_can_run_ahead`); its token ids then come straight from the
        sampler's device buffer.  Otherwise the call first reads the ids and
        plans as usual."""
        finished: List[Request] = []
        if self._inflight is not None and self._can_run_ahead():
            prev = self._inflight
            try:
                self._inflight = self._launch(prev.plan, ahead_of=prev)
            except (OutOfPages, OutOfSlots):
                self._inflight = None                          # no room: nothing was taken; plan again below
            finished += self._harvest(prev)
            if self._inflight is not None:
                self.scheduler.stats["steps_run_ahead"] = self.scheduler.stats.get("steps_run_ahead", 0) + 1
                if finished:
                    ops.check_device_errors(self.engine_config.device)    # as below: no tokens of a failed step
                return [self._result(r) for r in finished]
        elif self._inflight is not None:
            prev, self._inflight = self._inflight, None
            finished += self._harvest(prev)
        plan = self.scheduler.schedule()
        finished += plan.finished
        if plan.items:
            self.scheduler.begin_step(plan)
            self._inflight = self._launch(plan)
            if not self.engine_config.pipeline_decode:
                prev, self._inflight = self._inflight, None
                finished += self._harvest(prev)
        if finished:
            ops.check_device_errors(self.engine_config.device)    # a kernel's bounded wait ran out: do not hand out its tokens
        return [self._result(r) for r in finished]

    def _launch(self, plan: StepPlan, ahead_of: Optional["_Launched"] = None) -> "_Launched":
        """Start a step: run the plan's tokens, sample, start the copy of the ids
        to the host.  ``ahead_of``: the step before this one, not yet read; the
        plan is that step's (the same decoding requests, one token further)."""
        if ahead_of is not None:
            reqs = [it.request for it in plan.items]
            entries = [StepEntry(r.rid, [0], [0]) for r in reqs]
            logits = self.runner.step(entries, device_tokens=ahead_of.ids)
            plan = StepPlan(items=[Planned(r, r.computed + 1, 1, True) for r in reqs])
            sampling, extra = reqs, 1
        else:
            entries = []
            for it in plan.items:
                toks = it.request.token_slice(it.start, it.count)
                entries.append(StepEntry(it.request.rid, toks, [it.count - 1] if it.samples else []))
            logits = self.runner.step(entries)
            sampling, extra = [it.request for it in plan.items if it.samples], 0
        ids, host, event = None, None, None
        if sampling:
            slots = [self.runner.slots.slot(r.rid) for r in sampling]
            for r, slot in zip(sampling, slots):
                # a request that samples for the first time (or again after giving way) has all its tokens on the
                # host: its ring of recent tokens starts from them; from then on the sampler appends on the device
                if self.sampler.serves_from_ring(r.params) and self._ring_seeded.get(r.rid) != r.preemptions:
                    self.sampler.seed_ring(slot, r.tokens)
                    self._ring_seeded[r.rid] = r.preemptions
            ids = self.sampler.sample(
                logits, [r.params for r in sampling], [r.seed for r in sampling],
                [len(r.output) + extra for r in sampling],
                [r.tokens if r.params.has_penalties and not self.sampler.serves_from_ring(r.params) else ()
                 for r in sampling], slots)
            host = self._id_buffers[self._id_turn][:len(sampling)]
            self._id_turn ^= 1
            host.copy_(ids, non_blocking=True)
            event = torch.cuda.Event()
            event.record()
        return _Launched(plan, sampling, ids, host, event)

    def _harvest(self, done: "_Launched") -> List[Request]:
        """Wait for a started step's ids and record the step.  Requests that
        finished while it was already running (it was started ahead) are
        skipped: their extra token is dropped."""
        sampled: Dict[Hashable, int] = {}
        if done.event is not None:
            done.event.synchronize()
            for r, t in zip(done.sampling, done.host.tolist()):
                sampled[r.rid] = t
        plan = done.plan
        if any(it.request.phase is Phase.FINISHED for it in plan.items):
            plan = StepPlan(items=[it for it in plan.items if it.request.phase is not Phase.FINISHED])
        finished = self.scheduler.finish_step(plan, sampled)
        for r in finished:
            self._ring_seeded.pop(r.rid, None)
        return finished

    def _can_run_ahead(self) -> bool:
        """Whether the step after the one in flight is known before that one's
        ids are: it was a step of decoding requests only, nobody else waits or
        runs, none of them reaches its token or length limit with the id it is
        about to get, and none needs its recent tokens on the host (penalties
        over a window longer than the sampler's rings on the device).
        A request that stops on an end or stop token is found out one step
        late; that step's token for it is dropped."""
        if not self.engine_config.pipeline_decode:
            return False
        prev = self._inflight
        sch = self.scheduler
        if sch.waiting or len(prev.plan.items) != len(sch.running) or len(prev.sampling) != len(prev.plan.items):
            return False
        for it in prev.plan.items:
            r = it.request
            if it.count != 1 or not it.samples or r.phase is not Phase.RUNNING:
                return False
            if r.params.has_penalties and not self.sampler.serves_from_ring(r.params):
                return False
            if len(r.output) + 2 > r.params.max_tokens or len(r.prompt) + len(r.output) + 2 > self.runner.max_model_len:
                return False
        return True

    def _result(self, r: Request) -> GenerationResult:
        return GenerationResult(r.rid, len(r.prompt), list(r.output), r.finish_reason or "", r.preemptions)

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[GenerationResult]:
        """Generate for every prompt (lists of token ids); results in prompt order."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams per prompt (or one for all)")
        rids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        guard = 0
        # The collector of reference cycles is held off while the steps run: a step makes a few hundred small
        # containers, which set it off again and again, and with the prompts' token lists alive a full
        # collection takes tens of milliseconds, as long as ten decode steps.  (What a step makes is freed by
        # its reference counts.)
        collecting = gc.isenabled()
        gc.disable()
        try:
            while self.has_work():
                self.step()
                guard += 1
                if guard > 10_000_000:
                    raise RuntimeError("generation made no progress")
        finally:
            if collecting:
                gc.enable()
        return [self._result(self._requests[rid]) for rid in rids]

    def run_step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """The bare step function (no scheduling, no sampling): logits at the wanted places."""
        return self.runner.step(entries)

    def end_request(self, rid: Hashable) -> None:
        if self.runner.has(rid):
            self.runner.end(rid)

    @property
    def stats(self) -> dict:
        ops.check_device_errors(self.engine_config.device)
        s = dict(self.scheduler.stats)
        s.update(pages_free=[p.num_free for p in self.runner.kv.pools],
                 pages_total=[p.num_pages for p in self.runner.kv.pools],
                 page_reuses=[p.reuses for p in self.runner.kv.pools],
                 runner_steps=self.runner.steps, runner_tokens=self.runner.tokens_run)
        return s


def _require_cuda(device: str) -> None:
    if torch.device(device).type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError(f"inferflux_b200 runs on a CUDA device only (asked for '{device}', "
                           f"cuda available: {torch.cuda.is_available()}); there is no CPU path")
