"""Slots for per-request state of fixed size.

Every live request owns one slot for its whole life.  Mixers that carry state
across steps (a recurrence, a convolution tail) declare
:class:`~inferflux_b200.parts.base.StateNeed` entries and get, per run, one
tensor ``[max_seqs, *shape]`` indexed by slot; a slot's state is zeroed when a
request takes it.  An architecture whose mixers keep everything in pages
(grouped-query attention) declares none, and the slot is only the request's
seat.

The reference's counterpart is its 128 generation-stamped sequence leases
(runtime/scheduler/sequence_slot_manager.h:107-342) plus a device metadata
slab ``[token | n_past | seq_id | kv_len] x max_batch``
(runtime/backends/cuda/native/transformer_forward.cu:1112-1127).
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Sequence


class OutOfSlots(RuntimeError):
    pass


class StateSlotManager:
    """Host-side: which request sits in which slot."""

    def __init__(self, max_seqs: int):
        if max_seqs < 1:
            raise ValueError("max_seqs must be >= 1")
        self.max_seqs = max_seqs
        self._free: List[int] = list(range(max_seqs - 1, -1, -1))
        self._slot_of: Dict[Hashable, int] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    def has(self, rid: Hashable) -> bool:
        return rid in self._slot_of

    def slot(self, rid: Hashable) -> int:
        return self._slot_of[rid]

    def acquire(self, rid: Hashable) -> int:
        if rid in self._slot_of:
            raise KeyError(f"request {rid!r} already has a slot")
        if not self._free:
            raise OutOfSlots(f"all {self.max_seqs} state slots are taken")
        s = self._free.pop()
        self._slot_of[rid] = s
        return s

    def release(self, rid: Hashable) -> int:
        s = self._slot_of.pop(rid)
        self._free.append(s)
        return s

    def check(self) -> None:
        used = list(self._slot_of.values())
        assert len(set(used)) == len(used), "a slot is held twice"
        assert len(set(self._free)) == len(self._free), "a slot is twice in the free list"
        assert not set(used) & set(self._free), "a slot is free and held"
        assert len(used) + len(self._free) == self.max_seqs, "a slot was lost"


class StateSlotStorage:
    """Device-side: the state tensors of every run, ``[max_seqs, *shape]``."""

    def __init__(self, max_seqs: int, needs_per_run: Sequence[Sequence], device: str):
        import torch
        self.max_seqs = max_seqs
        self.tensors: List[Dict[str, "torch.Tensor"]] = []
        for needs in needs_per_run:
            self.tensors.append({n.name: torch.zeros((max_seqs, *n.shape), dtype=n.dtype, device=device)
                                 for n in needs})

    def of_run(self, run: int) -> Dict[str, "torch.Tensor"]:
        return self.tensors[run]

    def reset(self, slot: int) -> None:
        for per_run in self.tensors:
            for t in per_run.values():
                t[slot].zero_()

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for d in self.tensors for t in d.values())
