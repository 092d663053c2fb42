"""Choosing the next token of each request from its logits row, on the GPU.

Order per row, as in the reference (runtime/backends/cuda/inferflux_cuda_executor.cpp:2903-2932):
penalties over the recent tokens, then greedy argmax or a temperature draw.
Rows of one step are handled by one launch per kernel; a row's result depends
only on its own logits, parameters, seed and token index, never on the batch.

The recent tokens that the penalties count live on the device, in a ring per
state slot (the request's seat): the engine seeds a request's ring with its
prompt when the request first samples, and every sampled token is appended by
a kernel, so a step can be sampled before the host has seen the token of the
step before it.  The reference keeps the last 64 ids of every sequence on the
host (runtime/backends/cuda/inferflux_cuda_executor.h:310-313).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..kernels import ops
from .params import SamplingParams


class Sampler:
    RING = 256            # tokens a request's ring holds: the longest penalty window served from the device

    def __init__(self, vocab_size: int, device: str, seed: int = 0, max_seqs: int = 0):
        self.vocab = vocab_size
        self.device = device
        self._rng = torch.Generator().manual_seed(seed)
        self._weights: Optional[torch.Tensor] = None
        self.max_seqs = max_seqs
        self._ring: Optional[torch.Tensor] = None        # int32 [max_seqs, RING], made at the first use
        self._ring_totals: Optional[torch.Tensor] = None

    # ------------------------------------------------------------- rings
    def _rings(self):
        if self._ring is None:
            self._ring = torch.zeros((self.max_seqs, self.RING), dtype=torch.int32, device=self.device)
            self._ring_totals = torch.zeros(self.max_seqs, dtype=torch.int32, device=self.device)
        return self._ring, self._ring_totals

    def seed_ring(self, slot: int, tokens: Sequence[int]) -> None:
        """The request in ``slot`` starts (again) with these tokens behind it."""
        ring, totals = self._rings()
        tail = list(tokens)[-self.RING:]
        if tail:
            ring[slot, :len(tail)].copy_(torch.tensor(tail, dtype=torch.int32), non_blocking=True)
        totals[slot:slot + 1].fill_(len(tail))

    def serves_from_ring(self, params: SamplingParams) -> bool:
        return self.max_seqs > 0 and params.has_penalties and params.penalty_last_n <= self.RING

    def fresh_seed(self) -> int:
        """A seed for a request that brought none."""
        return int(torch.randint(0, 2 ** 62, (1,), generator=self._rng))

    def _scratch(self, rows: int) -> torch.Tensor:
        need = rows * self.vocab
        if self._weights is None or self._weights.numel() < need:
            self._weights = torch.empty(need, dtype=torch.float32, device=self.device)
        return self._weights

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               counters: Sequence[int], recent: Sequence[Sequence[int]],
               slots: Optional[Sequence[int]] = None) -> torch.Tensor:
        """logits float32 [R, V] (changed in place by penalties); one token per
        row as an int32 device tensor.  ``counters[r]`` = how many tokens the
        request has sampled before; ``recent[r]`` = its latest tokens (prompt
        and output), of which the last ``penalty_last_n`` count.  With
        ``slots`` (the requests' state slots, rings seeded by
        :meth:`seed_ring`) the penalties are taken from the rings instead, and
        the sampled tokens are appended to them; ``recent`` is not read."""
        r = logits.shape[0]
        out = torch.empty(r, dtype=torch.int32, device=self.device)
        if r == 0:
            return out
        dev = self.device
        on_ring = [slots is not None and self.serves_from_ring(p) for p in params]
        on_host = [p.has_penalties and not ring for p, ring in zip(params, on_ring)]
        if any(on_host):                                     # windows too long for the rings: counted here, on the host
            width = max(1, max(min(p.penalty_last_n, len(rc)) if h else 0 for p, rc, h in zip(params, recent, on_host)))
            ids = torch.zeros((r, width), dtype=torch.int32)
            cnt = torch.zeros((r, width), dtype=torch.int32)
            n = torch.zeros(r, dtype=torch.int32)
            for i, (p, rc) in enumerate(zip(params, recent)):
                if not on_host[i]:
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
                                f([p.repetition_penalty if h else 1.0 for p, h in zip(params, on_host)]),
                                f([p.frequency_penalty if h else 0.0 for p, h in zip(params, on_host)]),
                                f([p.presence_penalty if h else 0.0 for p, h in zip(params, on_host)]))
        if not any(on_ring):
            return self._draw(logits, params, seeds, counters, out)
        ring, totals = self._rings()
        f = lambda vals, dt: torch.tensor(vals, dtype=dt).to(dev, non_blocking=True)
        d_slots = f([s if g else -1 for s, g in zip(slots, on_ring)], torch.int32)
        ops.apply_penalties_ring(logits, ring, totals, d_slots,
                                 f([p.penalty_last_n for p in params], torch.int32),
                                 f([p.repetition_penalty if g else 1.0 for p, g in zip(params, on_ring)], torch.float32),
                                 f([p.frequency_penalty if g else 0.0 for p, g in zip(params, on_ring)], torch.float32),
                                 f([p.presence_penalty if g else 0.0 for p, g in zip(params, on_ring)], torch.float32))
        self._draw(logits, params, seeds, counters, out)
        ops.ring_append(ring, totals, d_slots, out)
        return out

    def _draw(self, logits, params, seeds, counters, out) -> torch.Tensor:
        r, dev = logits.shape[0], self.device
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
