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

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..config import EngineConfig, ModelConfig, build_spec, load_config
from ..kernels import ops
from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .model import Model
from .runner import StepRunner, torch_dtype
from .scheduler import CacheView, Phase, Request, Scheduler, StepPlan


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
        self.sampler = Sampler(model.spec.vocab_size, engine_config.device, engine_config.seed)
        self._next_id = 0
        self._requests: Dict[Hashable, Request] = {}

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
                    **engine_options) -> "Engine":
        """A model of ``config``'s architecture with random weights from ``seed``,
        made directly on the device (no folder is written)."""
        from ..weights.random_init import random_tensors
        ecfg = EngineConfig(dtype=dtype, **engine_options)
        ecfg.validate()
        _require_cuda(ecfg.device)
        if isinstance(config, dict):
            config = load_config(config)
        td = torch_dtype(dtype)
        model = Model(build_spec(config), td, ecfg.device)
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
        return self.scheduler.has_work()

    def step(self) -> List[GenerationResult]:
        """Plan one step, run it, sample; returns the requests finished by it."""
        plan = self.scheduler.schedule()
        finished = list(plan.finished)
        if plan.items:
            self.scheduler.begin_step(plan)
            entries = []
            for it in plan.items:
                toks = it.request.token_slice(it.start, it.count)
                entries.append(StepEntry(it.request.rid, toks, [it.count - 1] if it.samples else []))
            logits = self.runner.step(entries)
            sampling = [it.request for it in plan.items if it.samples]
            sampled: Dict[Hashable, int] = {}
            if sampling:
                ids = self.sampler.sample(
                    logits, [r.params for r in sampling], [r.seed for r in sampling],
                    [len(r.output) for r in sampling],
                    [r.tokens if r.params.has_penalties else () for r in sampling])
                for r, t in zip(sampling, ids.tolist()):
                    sampled[r.rid] = t
            finished += self.scheduler.finish_step(plan, sampled)
        if finished:
            ops.check_device_errors(self.engine_config.device)    # a kernel's bounded wait ran out: do not hand out its tokens
        return [self._result(r) for r in finished]

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
        while self.scheduler.has_work():
            self.step()
            guard += 1
            if guard > 10_000_000:
                raise RuntimeError("generation made no progress")
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
