"""Run-time settings of the engine (not of the model).

Names and defaults follow the reference's scheduler and KV settings where it
has them: ``max_batch_tokens`` 16384 and ``max_batch_size`` 32
(scheduler/scheduler.h:74-76), ``chunked_prefill_tokens`` 512 and
``mixed_prefill_budget_ratio`` (scheduler/scheduler.h:83-84,
runtime/execution/batch_executor.cpp:196-213), 16-token KV blocks
(scheduler/scheduler.cpp:138), 128 sequence slots (scheduler/scheduler.cpp:132).
The reference sizes its dense KV buffer from ``kv_max_batch`` x ``kv_max_seq``
(runtime/backends/cuda/native/native_bootstrap_config.h:8-29); the paged pool
here is sized in tokens (``kv_cache_tokens``) or as a fraction of free memory
(``kv_memory_ratio``, the reference's ratio knob,
runtime/backends/cuda/native/kv_cache_planner.h:76-127).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

DTYPES = ("bfloat16", "float32")


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"
    device: str = "cuda:0"
    page_size: int = 16
    kv_cache_tokens: Optional[int] = None   # pool size in tokens per cache group
    kv_memory_ratio: float = 0.80           # of free memory, when kv_cache_tokens is None
    max_seqs: int = 128                     # state slots = live requests
    max_batch_tokens: int = 16384           # tokens per step
    max_batch_size: int = 32                # requests per step
    chunked_prefill_tokens: int = 512       # most prompt tokens of one request per step
    mixed_prefill_budget_ratio: float = 1.0  # share of max_batch_tokens that prompts may take beside decodes
    max_model_len: Optional[int] = None     # default: the model's max_position_embeddings
    cuda_graphs: bool = True                # capture decode-only steps as CUDA graphs
    pipeline_decode: bool = True            # start a decode step before the one before it has reported its tokens
    seed: int = 0

    def validate(self) -> None:
        if self.dtype not in DTYPES:
            raise ValueError(f"dtype must be one of {DTYPES}, got '{self.dtype}'")
        if self.page_size < 1 or self.page_size & (self.page_size - 1):
            raise ValueError(f"page_size must be a power of two, got {self.page_size}")
        if self.max_seqs < 1:
            raise ValueError("max_seqs must be >= 1")
        if self.max_batch_tokens < 1 or self.max_batch_size < 1:
            raise ValueError("max_batch_tokens and max_batch_size must be >= 1")
        if self.chunked_prefill_tokens < 1:
            raise ValueError("chunked_prefill_tokens must be >= 1")
        if not 0.0 < self.mixed_prefill_budget_ratio <= 1.0:
            raise ValueError("mixed_prefill_budget_ratio must be in (0, 1]")
        if self.kv_cache_tokens is not None and self.kv_cache_tokens < self.page_size:
            raise ValueError("kv_cache_tokens must hold at least one page")
