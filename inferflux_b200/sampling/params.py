"""Per-request sampling parameters, with the reference's names, meanings and
defaults (``SamplingParams``, scheduler/request_batch.h:20-35; ``max_tokens``
256, request_batch.h:130):

temperature 1.0 (<= 0 = greedy), top_p 1.0 (off), top_k 0 (off), min_p 0.0
(off), frequency_penalty / presence_penalty 0.0, repetition_penalty 1.0 (off),
penalty_last_n 64 (how many recent tokens the penalties look at), seed (None =
unseeded: the engine draws one; the reference uses UINT32_MAX for that).

Differences from the reference's native sampler, on purpose: top_k and min_p
are applied (the reference accepts top_k and ignores it,
runtime/backends/cuda/native/gpu_sampler.cu:562-567); a greedy request gets no
hidden repetition penalty (the reference forces 1.15,
runtime/backends/cuda/inferflux_cuda_executor.cpp:2906-2910); a seeded request
draws a fresh uniform per token from (seed, token index) instead of re-seeding
the generator on every call (gpu_sampler.cu:603-605), which repeats one
uniform.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repetition_penalty: float = 1.0
    penalty_last_n: int = 64
    seed: Optional[int] = None
    max_tokens: int = 256
    stop_token_ids: List[int] = field(default_factory=list)
    ignore_eos: bool = False

    def validate(self) -> None:
        if self.top_p <= 0.0 or self.top_p > 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p}")
        if self.repetition_penalty <= 0.0:
            raise ValueError(f"repetition_penalty must be > 0, got {self.repetition_penalty}")
        if self.penalty_last_n < 0:
            raise ValueError("penalty_last_n must be >= 0")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def has_penalties(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0
                or self.presence_penalty != 0.0) and self.penalty_last_n > 0
