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

import torch

QUERY_TILE = 16     # tokens per query tile of the generic attention kernel
CHUNK_TILE = 64     # tokens per query tile of the mma.sync kernel for prompt portions
UMMA_TILE = 128     # tokens per query tile of the tcgen05 kernel for prompt portions


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens (a portion of its prompt
    or one decoded token) and the places among them whose logits are wanted."""

    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


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
            raise RuntimeError(f"step metadata needs {start + n} words, the slab holds {self.capacity}")
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
class StepContext:
    """What parts see of a step.  All tensors are int32 on the device."""

    n_tokens: int
    n_entries: int
    entries: List[StepEntry]                  # host view, in batch order
    ctx_starts: List[int]                     # host: tokens cached before each entry's new ones
    slots: List[int]                          # host: state slot of each entry
    token_ids: torch.Tensor                   # [N]
    positions: torch.Tensor                   # [N]
    entry_q_start: torch.Tensor               # [R] row of each entry's first new token
    entry_q_len: torch.Tensor                 # [R]
    entry_ctx_start: torch.Tensor             # [R]
    entry_slot: torch.Tensor                  # [R]
    tile_entry: torch.Tensor                  # [T] query tiles of QUERY_TILE tokens
    tile_q0: torch.Tensor                     # [T]
    n_tiles: int
    chunk_tile_entry: torch.Tensor            # [Tc] tiles of CHUNK_TILE tokens over entries with more than one token
    chunk_tile_q0: torch.Tensor               # [Tc]
    n_chunk_tiles: int
    umma_tile_entry: torch.Tensor             # [Tu] tiles of UMMA_TILE tokens over the same entries
    umma_tile_q0: torch.Tensor                # [Tu]
    n_umma_tiles: int
    decode_entries: torch.Tensor              # [D] entries that bring exactly one token
    n_decode: int
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
    position_tables: Dict[str, Tuple[torch.Tensor, torch.Tensor]] = field(default_factory=dict)
    extras: Dict[str, object] = field(default_factory=dict)
    decode_skewed: bool = False               # the single tokens' contexts differ much in length (contexts_skewed)

    def buffer(self, shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


def contexts_skewed(lengths) -> bool:
    """Whether the contexts of a step's single tokens differ so much in length
    that attention should share its work out by tiles and not by requests: the
    longest is at least 1,024 tokens and at least 1.5 times the mean.  With
    equal contexts the kernel that gives every request its own blocks is about
    a fifth faster; with one long context among short ones it takes as long as
    the long one alone."""
    n = len(lengths)
    if n < 2:
        return False
    longest = max(lengths)
    return longest >= 1024 and 2 * longest * n >= 3 * sum(lengths)
