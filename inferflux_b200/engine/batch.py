"""One step's input: a batch of (request, its next tokens), and the device-side
description of it that the kernels read.

The reference's step input is ``UnifiedBatchInput{sequence_id, n_past,
tokens, request_logits, ...}`` (runtime/backends/common/backend_types.h:19-28)
and its step splits a mixed batch into one batched decode forward plus one
forward per prompt portion
(runtime/backends/cuda/inferflux_cuda_executor.cpp:2806-2849,3041-3099).  Here
all entries are flattened into one token list and run as one batch; logits are
returned at the positions each entry asks for (the reference returns them for
the last token only, runtime/backends/cuda/native/transformer_forward.cu:2105-2112).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Sequence, Tuple

import numpy as np
import torch


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens (a portion of its prompt
    or one decoded token) and the places among them whose logits are wanted."""

    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


class SlabFull(RuntimeError):
    """The step's metadata does not fit the slab it is written into."""


class MetadataSlab:
    """All int32 metadata of a step in one pinned host buffer and one device
    buffer, so a step costs one host-to-device copy.

    The copy is asynchronous and the GPU may run several steps behind the
    host, so the host side is a small ring of pinned buffers: a buffer is
    written again only after the copy that last read it has completed (an
    event per buffer tells)."""

    RING = 4

    def __init__(self, capacity: int, device: str):
        self.capacity = capacity
        self.device = device
        self._cuda = torch.device(device).type == "cuda"
        n = self.RING if self._cuda else 1
        self._hosts = [torch.zeros(capacity, dtype=torch.int32, pin_memory=self._cuda) for _ in range(n)]
        self._events = [None] * n
        self._turn = -1
        self.host = self._hosts[0]
        self._np = self.host.numpy()
        self.dev = torch.zeros(capacity, dtype=torch.int32, device=device)
        self._used = 0

    def begin(self) -> None:
        self._turn = (self._turn + 1) % len(self._hosts)
        ev = self._events[self._turn]
        if ev is not None:
            ev.synchronize()            # the copy that read this buffer last has finished
        self.host = self._hosts[self._turn]
        self._np = self.host.numpy()
        self._used = 0

    def put(self, values, align: int = 4) -> torch.Tensor:
        """Append values; returns the device view (valid after :meth:`upload`)."""
        n = len(values)
        start = (self._used + align - 1) // align * align
        if start + n > self.capacity:
            raise SlabFull(f"step metadata needs {start + n} words, the slab holds {self.capacity}")
        if n:
            self._np[start:start + n] = values
        self._used = start + n
        return self.dev[start:start + n]

    def upload(self) -> None:
        if self._used:
            self.dev[:self._used].copy_(self.host[:self._used], non_blocking=True)
            if self._cuda:
                ev = self._events[self._turn]
                if ev is None:
                    ev = self._events[self._turn] = torch.cuda.Event()
                ev.record()


@dataclass
class StepLayout:
    """The shape of a step on the host, from which parts derive the metadata of
    their own kernels (:meth:`~inferflux_b200.parts.base.Part.describe_step`)."""

    n_entries: int
    n_tokens: int
    page_size: int
    q_len: np.ndarray                         # [R] new tokens of each entry
    q_start: np.ndarray                       # [R] row of each entry's first new token
    ctx_start: np.ndarray                     # [R] tokens cached before each entry's new ones


@dataclass
class StepContext:
    """What parts see of a step.  All tensors are int32 on the device.  What
    only one kind of part needs (the tile lists of the attention kernels, say)
    is not here but in ``extras`` under that part's ``describe_key``."""

    n_tokens: int
    n_entries: int
    entries: List[StepEntry]                  # host view, in batch order
    ctx_starts: List[int]                     # host: tokens cached before each entry's new ones
    slots: List[int]                          # host: state slot of each entry
    layout: StepLayout
    token_ids: torch.Tensor                   # [N]
    positions: torch.Tensor                   # [N]
    entry_q_start: torch.Tensor               # [R] row of each entry's first new token
    entry_q_len: torch.Tensor                 # [R]
    entry_ctx_start: torch.Tensor             # [R]
    entry_slot: torch.Tensor                  # [R]
    block_tables: List[torch.Tensor]          # per cache group [R, max_blocks]
    slot_maps: List[torch.Tensor]             # per cache group [N]
    want_rows: torch.Tensor                   # [W] rows whose logits are wanted
    n_want: int
    max_q_len: int
    max_ctx_len: int                          # longest context (cached + new) of any entry
    page_size: int
    kv: object                                # KVCacheStorage
    dtype: torch.dtype
    device: str
    position_tables: Dict[str, object] = field(default_factory=dict)   # position name -> what its prepare() returned
    extras: Dict[str, object] = field(default_factory=dict)            # describe_key -> what describe_step() returned

    def buffer(self, shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)
