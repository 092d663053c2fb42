"""The paged key/value cache: groups of runs with the same needs, a block
table per request and group, and the rules by which pages come and go.

A *group* holds the runs (layer executions) whose mixers ask for the same
:class:`~inferflux_b200.parts.base.KVNeed` (what a token caches: streams of
``heads x width`` elements, and a window).  Each group has a page pool of its
own; one page holds ``page_size`` tokens of every run of the group, laid out
``[page][run][stream][head][slot][width]`` so that one (page, run, stream,
head) tile is contiguous.  For attention the streams are keys and values of
equal shape, which gives ``[page][run][k|v][kv_head][slot][head_dim]``.

Pages are taken before a step for the tokens the step brings
(:meth:`KVCacheManager.reserve`), and given back when the request ends
(:meth:`free_request`) or, in a group with a window, once no later token can
see them (:meth:`advance`).  The manager is host-side bookkeeping and has no
GPU dependency; :class:`KVCacheStorage` owns the device tensors.

The reference sizes a dense buffer ``[max_batch][layers][2][max_seq][kv_dim]``
(runtime/backends/cuda/native/kv_cache_gpu.cu:32-38), clears a whole slot when
a sequence ends (runtime/backends/cuda/inferflux_cuda_executor.cpp:3467-3617)
and reserves ``ceil(prompt/16) + 1`` host-side blocks per request
(scheduler/scheduler.cpp:1827-1839).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

from ..parts.base import KVNeed
from .page_pool import OutOfPages, PagePool


@dataclass
class _Sequence:
    length: int = 0                    # tokens whose keys and values are in the cache
    reserved: int = 0                  # tokens for which pages are held (>= length)
    tables: List[List[int]] = field(default_factory=list)   # per group: page of each logical block, -1 = given back
    serial: int = 0                    # unique among all sequences the manager ever held
    version: int = 0                   # counts the changes of the block tables


class KVCacheManager:
    def __init__(self, needs: Sequence[KVNeed], num_pages: Sequence[int], page_size: int):
        if page_size < 1 or page_size & (page_size - 1):
            raise ValueError("page_size must be a power of two")
        if len(needs) != len(num_pages):
            raise ValueError("one pool size per cache group")
        self.needs = list(needs)
        self.page_size = page_size
        self.pools = [PagePool(n, g) for g, n in enumerate(num_pages)]
        self._seqs: Dict[Hashable, _Sequence] = {}
        self._serials = 0

    # ------------------------------------------------------------ queries
    @property
    def num_groups(self) -> int:
        return len(self.needs)

    def has(self, rid: Hashable) -> bool:
        return rid in self._seqs

    def length(self, rid: Hashable) -> int:
        return self._seqs[rid].length

    def num_free(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def block_table(self, rid: Hashable, group: int) -> List[int]:
        return self._seqs[rid].tables[group]

    def table_stamp(self, rid: Hashable):
        """Changes whenever the request's block tables do (a page taken or given
        back, or the request ended and begun again), so a copy of the tables
        made under the same stamp is still right."""
        seq = self._seqs[rid]
        return (seq.serial, seq.version)

    def _first_needed_block(self, group: int, length: int) -> int:
        """Blocks below this one lie wholly behind the window of every token at
        position >= length."""
        w = self.needs[group].window
        if not w:
            return 0
        first_key = max(0, length - w + 1)
        return first_key // self.page_size

    def pages_needed(self, rid: Optional[Hashable], n_new: int, cached: Optional[int] = None) -> List[int]:
        """Pages each group must still hand out so that ``n_new`` more tokens
        fit (for a request not yet known, give ``cached`` = 0)."""
        if rid is not None and rid in self._seqs:
            seq = self._seqs[rid]
            have = [len(t) for t in seq.tables]
            end = seq.length + n_new
        else:
            have = [0] * self.num_groups
            end = (cached or 0) + n_new
        blocks = (end + self.page_size - 1) // self.page_size
        return [max(0, blocks - h) for h in have]

    def can_reserve(self, rid: Optional[Hashable], n_new: int) -> bool:
        return all(n <= self.pools[g].num_free for g, n in enumerate(self.pages_needed(rid, n_new)))

    # ------------------------------------------------------------ changes
    def add_request(self, rid: Hashable) -> None:
        if rid in self._seqs:
            raise KeyError(f"request {rid!r} is already in the cache")
        self._serials += 1
        self._seqs[rid] = _Sequence(tables=[[] for _ in self.needs], serial=self._serials)

    def reserve(self, rid: Hashable, n_new: int) -> None:
        """Hold pages for positions [length, length + n_new) in every group, or
        raise :class:`OutOfPages` and hold nothing new."""
        seq = self._seqs[rid]
        need = self.pages_needed(rid, n_new)
        for g, n in enumerate(need):
            if n > self.pools[g].num_free:
                raise OutOfPages(n, self.pools[g].num_free, g)
        for g, n in enumerate(need):
            if n:
                seq.tables[g].extend(self.pools[g].alloc(n))
                seq.version += 1
        seq.reserved = max(seq.reserved, seq.length + n_new)

    def advance(self, rid: Hashable, n_new: int) -> None:
        """The step wrote ``n_new`` tokens: move the length on and give back the
        pages that a window has passed."""
        seq = self._seqs[rid]
        if seq.length + n_new > seq.reserved:
            raise RuntimeError(f"request {rid!r}: advance beyond the reserved pages")
        seq.length += n_new
        for g in range(self.num_groups):
            first = self._first_needed_block(g, seq.length)
            table = seq.tables[g]
            gone = [table[b] for b in range(min(first, len(table))) if table[b] >= 0]
            if gone:
                for b in range(min(first, len(table))):
                    table[b] = -1
                self.pools[g].free(gone)
                seq.version += 1

    def free_request(self, rid: Hashable) -> None:
        seq = self._seqs.pop(rid)
        for g, table in enumerate(seq.tables):
            self.pools[g].free([p for p in table if p >= 0])

    def slot_of(self, rid: Hashable, group: int, position: int) -> int:
        """page * page_size + offset of a position's keys and values."""
        page = self._seqs[rid].tables[group][position // self.page_size]
        if page < 0:
            raise RuntimeError(f"request {rid!r}: position {position} lies in a page that was given back")
        return page * self.page_size + position % self.page_size

    def check(self) -> None:
        """Every held page is in exactly one block table; pools are consistent."""
        for g, pool in enumerate(self.pools):
            pool.check()
            held = [p for s in self._seqs.values() for p in s.tables[g] if p >= 0]
            assert len(held) == len(set(held)), f"group {g}: a page is in two block tables"
            assert len(held) == pool.num_held, f"group {g}: {pool.num_held} pages held, {len(held)} in tables"


class KVCacheStorage:
    """The device tensors of the cache groups."""

    def __init__(self, needs: Sequence[KVNeed], runs_per_group: Sequence[int], num_pages: Sequence[int],
                 page_size: int, dtype, device: str):
        import torch
        self.page_size = page_size
        self.needs = list(needs)
        self.pools = []
        for need, n_runs, pages in zip(needs, runs_per_group, num_pages):
            # zeros, not empty: a masked key is multiplied by 0, which must not meet a NaN
            self.pools.append(torch.zeros((pages, n_runs, page_size * need.elements_per_token),
                                          dtype=dtype, device=device))

    def stream_views(self, group: int, index: int):
        """For one run: {stream name: its ``[heads, page_size, width]`` block
        inside page 0}, and the number of elements between pages.  Page p's
        block lies ``p * stride`` elements further on."""
        import torch
        pool, ps = self.pools[group], self.page_size
        views, at = {}, pool[0, index].storage_offset()
        for s in self.needs[group].streams:
            views[s.name] = torch.as_strided(pool, (s.heads, ps, s.width), (ps * s.width, s.width, 1), at)
            at += s.heads * ps * s.width
        return views, pool.stride(0)

    def layer_views(self, group: int, index: int):
        """(keys of page 0, values of page 0, elements between pages) of one run
        whose streams are ``k`` and ``v``."""
        views, stride = self.stream_views(group, index)
        return views["k"], views["v"], stride

    def bytes(self) -> int:
        return sum(p.numel() * p.element_size() for p in self.pools)


def bytes_per_token(needs: Sequence[KVNeed], runs_per_group: Sequence[int], element_size: int) -> int:
    """Cache bytes one token takes over all groups: runs * elements of all
    streams * element size each; for keys and values that is 2 * runs *
    kv_heads * head_dim (the reference's planner has the same product,
    runtime/backends/cuda/native/kv_cache_planner.h:22-37)."""
    return sum(r * n.elements_per_token * element_size for n, r in zip(needs, runs_per_group))
