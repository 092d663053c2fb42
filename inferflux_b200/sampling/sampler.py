"""Choosing the next token of each request from its logits row, on the GPU.

Order per row, as in the reference (runtime/backends/cuda/inferflux_cuda_executor.cpp:2903-2932):
penalties over the recent tokens, then greedy argmax or a temperature draw.
Rows of one step are handled by one launch per kernel; a row's result depends
only on its own logits, parameters, seed and token index, never on the batch.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..kernels import ops
from .params import SamplingParams


class Sampler:
    def __init__(self, vocab_size: int, device: str, seed: int = 0):
        self.vocab = vocab_size
        self.device = device
        self._rng = torch.Generator().manual_seed(seed)
        self._weights: Optional[torch.Tensor] = None

    def fresh_seed(self) -> int:
        """A seed for a request that brought none."""
        return int(torch.randint(0, 2 ** 62, (1,), generator=self._rng))

    def _scratch(self, rows: int) -> torch.Tensor:
        need = rows * self.vocab
        if self._weights is None or self._weights.numel() < need:
            self._weights = torch.empty(need, dtype=torch.float32, device=self.device)
        return self._weights

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               counters: Sequence[int], recent: Sequence[Sequence[int]]) -> torch.Tensor:
        """logits float32 [R, V] (changed in place by penalties); one token per
        row as an int32 device tensor.  ``counters[r]`` = how many tokens the
        request has sampled before; ``recent[r]`` = its latest tokens (prompt
        and output), of which the last ``penalty_last_n`` count."""
        r = logits.shape[0]
        out = torch.empty(r, dtype=torch.int32, device=self.device)
        if r == 0:
            return out
        dev = self.device
        if any(p.has_penalties for p in params):
            width = max(1, max(min(p.penalty_last_n, len(rc)) if p.has_penalties else 0
                               for p, rc in zip(params, recent)))
            ids = torch.zeros((r, width), dtype=torch.int32)
            cnt = torch.zeros((r, width), dtype=torch.int32)
            n = torch.zeros(r, dtype=torch.int32)
            for i, (p, rc) in enumerate(zip(params, recent)):
                if not p.has_penalties:
                    continue
                counts = {}
                for t in list(rc)[-p.penalty_last_n:]:
                    counts[int(t)] = counts.get(int(t), 0) + 1
                for k, (t, c) in enumerate(counts.items()):
                    ids[i, k], cnt[i, k] = t, c
                n[i] = len(counts)
            f = lambda vals: torch.tensor(vals, dtype=torch.float32).to(dev, non_blocking=True)
            ops.apply_penalties(logits, ids.to(dev, non_blocking=True), cnt.to(dev, non_blocking=True),
                                n.to(dev, non_blocking=True),
                                f([p.repetition_penalty if p.has_penalties else 1.0 for p in params]),
                                f([p.frequency_penalty if p.has_penalties else 0.0 for p in params]),
                                f([p.presence_penalty if p.has_penalties else 0.0 for p in params]))
        if all(p.greedy for p in params):
            return ops.argmax(logits, out)
        f = lambda vals, dt: torch.tensor(vals, dtype=dt).to(dev, non_blocking=True)
        ops.sample(logits, self._scratch(r),
                   f([p.temperature for p in params], torch.float32),
                   f([p.top_k for p in params], torch.int32),
                   f([p.top_p for p in params], torch.float32),
                   f([p.min_p for p in params], torch.float32),
                   f([s & 0x7FFFFFFFFFFFFFFF for s in seeds], torch.int64),
                   f(list(counters), torch.int64), out)
        return out
