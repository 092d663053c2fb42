"""The step function: run one batch of (request, its next tokens) from the
cache and return the logits at the wanted places.

:class:`StepRunner` owns the model, the cache (pages and state slots) and the
step metadata.  Generation (the scheduler and the Python entry point) and trace
replay both drive this one object; nothing else runs the model.

Reference counterpart: ``InferfluxCudaExecutor::ExecuteUnifiedBatch``
(runtime/backends/cuda/inferflux_cuda_executor.cpp:2743-3226), which splits a
mixed batch into a decode forward and one forward per prompt portion and
returns sampled tokens; here the whole batch is one forward and the result is
logits.
"""
from __future__ import annotations

from typing import Hashable, Optional, Sequence

import numpy as np
import torch

from ..cache import OutOfPages, OutOfSlots, KVCacheManager, KVCacheStorage, StateSlotManager, StateSlotStorage, bytes_per_token
from ..config.engine_config import EngineConfig
from .batch import MetadataSlab, SlabFull, StepContext, StepEntry, StepLayout
from ..kernels import ops
from .model import Model

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def torch_dtype(name: str) -> torch.dtype:
    try:
        return _TORCH_DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_TORCH_DTYPES)}, got '{name}'") from None


class StepRunner:
    def __init__(self, model: Model, engine_config: EngineConfig):
        engine_config.validate()
        self.model = model
        self.cfg = engine_config
        self.device = engine_config.device
        self.dtype = model.dtype
        self.page_size = engine_config.page_size
        self.max_model_len = engine_config.max_model_len or model.spec.max_position
        needs = model.kv_needs
        elt = torch.empty((), dtype=self.dtype).element_size()
        per_token = max(1, bytes_per_token(needs, model.runs_per_group, elt))
        if engine_config.kv_cache_tokens is not None:
            tokens = engine_config.kv_cache_tokens
        else:
            free, _ = torch.cuda.mem_get_info(torch.device(self.device))
            tokens = int(free * engine_config.kv_memory_ratio) // per_token
            tokens = min(tokens, engine_config.max_seqs * self.max_model_len)
        pages = max(1, (tokens + self.page_size - 1) // self.page_size)
        self.num_pages = [pages for _ in needs]
        self.kv = KVCacheManager(needs, self.num_pages, self.page_size)
        self.kv_storage = KVCacheStorage(needs, model.runs_per_group, self.num_pages, self.page_size,
                                         self.dtype, self.device)
        self.slots = StateSlotManager(engine_config.max_seqs)
        self.state_storage = StateSlotStorage(engine_config.max_seqs, model.state_needs, self.device)
        model.attach_states(self.state_storage)
        self.slab = MetadataSlab(1 << 16, self.device)
        self._graphs = {}
        self._capture_stream = None
        self._graph_pool = None
        self._graph_uses = {}
        self.graph_replays = 0
        self.steps = 0
        self.tokens_run = 0

    # ------------------------------------------------------------ requests
    def has(self, rid: Hashable) -> bool:
        return self.kv.has(rid)

    def length(self, rid: Hashable) -> int:
        return self.kv.length(rid)

    def begin(self, rid: Hashable) -> None:
        """Seat a new request: a state slot (zeroed) and empty block tables."""
        slot = self.slots.acquire(rid)
        self.kv.add_request(rid)
        self.state_storage.reset(slot)

    def end(self, rid: Hashable) -> None:
        """The request is finished: its pages and its slot are given back."""
        self.kv.free_request(rid)
        self.slots.release(rid)

    def can_run(self, rid: Optional[Hashable], n_new: int) -> bool:
        """Whether pages (and, for an unknown request, a slot) for ``n_new`` more tokens exist."""
        if (rid is None or not self.kv.has(rid)) and self.slots.num_free == 0:
            return False
        return self.kv.can_reserve(rid, n_new)

    # ---------------------------------------------------------------- step
    def _admit(self, entries: Sequence[StepEntry], check_tokens: bool = True) -> list:
        """Check the entries, seat new requests and hold pages for the step's
        tokens; raises before anything is taken when they do not fit.  Returns
        the requests that this call seated."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        vocab = self.model.spec.vocab_size
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise ValueError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.rid!r}: an entry needs at least one token")
            if check_tokens and (min(e.tokens) < 0 or max(e.tokens) >= vocab):
                raise ValueError(f"request {e.rid!r}: a token id is outside the vocabulary [0, {vocab})")
            for p in e.want:
                if not 0 <= int(p) < len(e.tokens):
                    raise ValueError(f"request {e.rid!r}: wanted place {p} is outside its {len(e.tokens)} tokens")
        new = [e for e in entries if not self.kv.has(e.rid)]
        if len(new) > self.slots.num_free:
            raise OutOfSlots(f"{len(new)} new request(s) but {self.slots.num_free} free state slot(s)")
        total = [0] * self.kv.num_groups
        for e in entries:
            known = self.kv.has(e.rid)
            have = self.kv.length(e.rid) if known else 0
            if have + len(e.tokens) > self.max_model_len:
                raise ValueError(f"request {e.rid!r}: {have + len(e.tokens)} tokens exceed "
                                 f"the model length {self.max_model_len}")
            for g, k in enumerate(self.kv.pages_needed(e.rid if known else None, len(e.tokens), 0)):
                total[g] += k
        for g, k in enumerate(total):
            if k > self.kv.num_free(g):
                raise OutOfPages(k, self.kv.num_free(g), g)
        for e in new:
            self.begin(e.rid)
        for e in entries:
            self.kv.reserve(e.rid, len(e.tokens))
        return [e.rid for e in new]

    def _layout(self, entries: Sequence[StepEntry]) -> StepLayout:
        r = len(entries)
        lens = np.fromiter((len(e.tokens) for e in entries), dtype=np.int64, count=r)
        starts = np.fromiter((self.kv.length(e.rid) for e in entries), dtype=np.int64, count=r)
        q_start = np.zeros(r, dtype=np.int64)
        np.cumsum(lens[:-1], out=q_start[1:])
        return StepLayout(n_entries=r, n_tokens=int(lens.sum()), page_size=self.page_size, q_len=lens,
                          q_start=q_start, ctx_start=starts)

    def _describe(self, entries: Sequence[StepEntry], slab: Optional[MetadataSlab] = None,
                  widths: Optional[Sequence[int]] = None) -> StepContext:
        """Write the step's metadata into a slab (the runner's own unless one is
        given) and return the context whose tensors are views of it.  With
        ``widths`` the block tables are padded to those widths, so that steps
        of the same shape have the same layout.  The runner writes what every
        part needs (tokens, positions, entries, block tables, cache slots,
        wanted rows); parts that describe the step for their own kernels add to
        the same slab before it is copied."""
        if slab is not None:
            return self._describe_into(entries, slab, widths)
        while True:
            try:
                return self._describe_into(entries, self.slab, widths)
            except SlabFull:
                self.slab = MetadataSlab(2 * self.slab.capacity, self.device)

    def _describe_into(self, entries: Sequence[StepEntry], slab: MetadataSlab,
                       widths: Optional[Sequence[int]]) -> StepContext:
        ps = self.page_size
        layout = self._layout(entries)
        r, n, lens, starts, q_start = layout.n_entries, layout.n_tokens, layout.q_len, layout.ctx_start, layout.q_start
        token_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        entry_of_token = np.repeat(np.arange(r), lens)
        offs = np.arange(n) - q_start[entry_of_token]
        positions = starts[entry_of_token] + offs
        slots = [self.slots.slot(e.rid) for e in entries]
        want_rows = [int(q_start[i]) + int(p) for i, e in enumerate(entries) for p in e.want]
        groups = self.kv.num_groups
        tables, slot_maps, out_widths = [], [], []
        for g in range(groups):
            tabs = [self.kv.block_table(e.rid, g) for e in entries]
            width = max(1, max(len(t) for t in tabs))
            if widths is not None:
                if widths[g] < width:
                    raise RuntimeError("block tables are wider than the layout they are written into")
                width = widths[g]
            arr = np.full((r, width), -1, dtype=np.int32)
            for i, t in enumerate(tabs):
                arr[i, :len(t)] = t
            pages = arr[entry_of_token, positions // ps]
            slot_maps.append(pages.astype(np.int64) * ps + positions % ps)
            tables.append(arr.reshape(-1))
            out_widths.append(width)
        slab.begin()
        d_tok, d_pos = slab.put(token_ids), slab.put(positions)
        d_qs, d_ql, d_cs, d_sl = slab.put(q_start), slab.put(lens), slab.put(starts), slab.put(slots)
        d_want = slab.put(want_rows)
        d_tabs = [slab.put(t).view(r, w) for t, w in zip(tables, out_widths)]
        d_sm = [slab.put(sm) for sm in slot_maps]
        extras = self.model.describe_step(layout, slab.put)
        slab.upload()
        return StepContext(
            n_tokens=n, n_entries=r, entries=list(entries), ctx_starts=starts.tolist(), slots=slots, layout=layout,
            token_ids=d_tok, positions=d_pos, entry_q_start=d_qs, entry_q_len=d_ql, entry_ctx_start=d_cs,
            entry_slot=d_sl, block_tables=d_tabs, slot_maps=d_sm, want_rows=d_want, n_want=len(want_rows),
            max_q_len=int(lens.max()),
            max_ctx_len=int((starts + lens).max()) if widths is None else max(out_widths) * ps,
            page_size=ps, kv=self.kv_storage, dtype=self.dtype, device=self.device, extras=extras)

    def build_context(self, entries: Sequence[StepEntry]) -> StepContext:
        """Reserve pages for the step's tokens and describe the step on the device."""
        self._admit(entries)
        return self._describe(entries)

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run the entries' tokens as one batch; float32 logits ``[wanted, vocab]``
        in the order of the entries and of each entry's ``want``.  Raises
        :class:`~inferflux_b200.cache.OutOfPages` (before anything ran) when
        the pools cannot hold the step's tokens.  The logits of a decode-only
        step live in a buffer that the next such step overwrites.

        If describing or running the step raises (metadata that does not fit, a
        shape a kernel refuses), the requests that this call seated are ended
        again, so their slots and pages are back; requests known before keep
        the pages held for this step's tokens (their cached length is
        unchanged, the pages serve the next attempt) until they end.

        With ``device_tokens`` (int32 on the device, one per entry, every entry
        a single token) the token ids are taken from there instead of the
        entries: the ids a sampler has just written need not visit the host
        before the next step starts."""
        if device_tokens is not None and any(len(e.tokens) != 1 for e in entries):
            raise ValueError("device_tokens serve entries of one token each")
        seated = self._admit(entries, check_tokens=device_tokens is None)
        try:
            if self._graphable(entries):
                logits = self._step_graph(entries, device_tokens)
            else:
                ctx = self._describe(entries)
                if device_tokens is not None:
                    ctx.token_ids.copy_(device_tokens[:len(entries)])
                logits = self.model.forward(ctx)
        except BaseException:
            for rid in seated:
                self.end(rid)
            raise
        n = 0
        for e in entries:
            self.kv.advance(e.rid, len(e.tokens))
            n += len(e.tokens)
        self.steps += 1
        self.tokens_run += n
        return logits

    # ------------------------------------------------------- captured decode
    GRAPH_WIDTH_STEP = 32      # block-table widths of captured steps are multiples of this many pages
    MAX_GRAPHS = 48
    CAPTURE_ON_USE = 3         # a shape is captured when it comes the third time; before that its steps run eagerly

    def _graphable(self, entries: Sequence[StepEntry]) -> bool:
        """A step of single decoded tokens, each wanting its logits, runs as a
        captured CUDA graph (the same kernels, launched by one replay)."""
        if not self.cfg.cuda_graphs or torch.device(self.device).type != "cuda":
            return False
        return all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)

    def _step_graph(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        step = self.GRAPH_WIDTH_STEP
        widths = tuple((max(len(self.kv.block_table(e.rid, g)) for e in entries) + step - 1) // step * step
                       for g in range(self.kv.num_groups))
        # what else decides which kernels the parts launch (attention: how much the contexts differ) is part of the shape
        key = (len(entries), widths, self.model.step_shape(self._layout(entries)))
        rec = self._graphs.get(key)
        if rec is None:
            # While requests join and leave, many batch sizes come once or twice; capturing costs more than
            # running such a step eagerly.
            seen = self._graph_uses.get(key, 0) + 1
            self._graph_uses[key] = seen
            if seen < self.CAPTURE_ON_USE:
                if len(self._graph_uses) > 4096:
                    self._graph_uses.clear()
                ctx = self._describe(entries)
                if device_tokens is not None:
                    ctx.token_ids.copy_(device_tokens[:len(entries)])
                return self.model.forward(ctx)
            if len(self._graphs) >= self.MAX_GRAPHS:
                self._graphs.pop(next(iter(self._graphs)))
            r = len(entries)
            words = 64 + 16 * r + sum(r * w for w in widths) + 8 * (14 + len(widths))
            while True:                                      # a slab of this step's own, as large as its metadata
                slab = MetadataSlab(words, self.device)
                try:
                    ctx = self._describe(entries, slab, widths)
                    break
                except SlabFull:
                    words *= 2
            if device_tokens is not None:
                ctx.token_ids.copy_(device_tokens[:r])
            logits = self.model.forward(ctx)                 # this step runs eagerly (and warms the libraries up)
            graph = torch.cuda.CUDAGraph()
            launches = ops.launch_count
            # Recorded on a stream of its own between capture_begin and capture_end; nothing runs.  (The
            # library's context manager would also hand every cached block back to the driver first, which
            # the next prompt step then has to ask for again: several milliseconds each way.)
            # All the graphs draw on one pool of memory: they replay one after the other on one stream, so what
            # one needs between its kernels may lie where another's did, and a capture seldom has to ask the
            # driver for memory.  What a graph hands out (its logits) stays its own while the record lives.
            if self._capture_stream is None:
                self._capture_stream = torch.cuda.Stream(device=self.device)
                self._graph_pool = torch.cuda.graph_pool_handle()
            self._capture_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._capture_stream):
                graph.capture_begin(pool=self._graph_pool)
                try:
                    static_logits = self.model.forward(ctx)
                finally:
                    graph.capture_end()
            torch.cuda.current_stream().wait_stream(self._capture_stream)
            off = lambda t: int(t.storage_offset())
            self._graphs[key] = dict(slab=slab, graph=graph, logits=static_logits, used=slab._used,
                                     launches=ops.launch_count - launches,
                                     image=slab._np[:slab._used].copy(), stamps=[None] * r, widths=widths,
                                     at=dict(tok=off(ctx.token_ids), pos=off(ctx.positions),
                                             cs=off(ctx.entry_ctx_start), sl=off(ctx.entry_slot),
                                             tab=[off(t) for t in ctx.block_tables],
                                             sm=[off(t) for t in ctx.slot_maps]))
            return logits
        self._refresh_decode(entries, rec)
        if device_tokens is not None:
            at = rec["at"]["tok"]
            rec["slab"].dev[at:at + len(entries)].copy_(device_tokens[:len(entries)])
        rec["graph"].replay()
        ops.launch_count += rec["launches"]
        self.graph_replays += 1
        return rec["logits"]

    def _refresh_decode(self, entries: Sequence[StepEntry], rec: dict) -> None:
        """The metadata of a captured decode step, brought up to date in the
        host image that the record keeps and sent to the device.  Per entry
        only the token, the position and the cache slot of the new token
        change from step to step; a row of a block table is written again only
        when its request's tables have changed (the stamp tells)."""
        img, at, widths, stamps = rec["image"], rec["at"], rec["widths"], rec["stamps"]
        kv, ps = self.kv, self.page_size
        for i, e in enumerate(entries):
            rid = e.rid
            length = kv.length(rid)
            img[at["tok"] + i] = e.tokens[0]
            img[at["pos"] + i] = length
            img[at["cs"] + i] = length
            stamp = (rid, kv.table_stamp(rid))
            fresh = stamps[i] != stamp
            if fresh:
                stamps[i] = stamp
                img[at["sl"] + i] = self.slots.slot(rid)
            for g, w in enumerate(widths):
                base = at["tab"][g] + i * w
                if fresh:
                    table = kv.block_table(rid, g)
                    if len(table) > w:
                        raise RuntimeError("block tables are wider than the layout they are written into")
                    img[base:base + len(table)] = table
                    img[base + len(table):base + w] = -1
                img[at["sm"][g] + i] = int(img[base + length // ps]) * ps + length % ps
        slab = rec["slab"]
        slab.begin()
        slab.put(img)
        slab.upload()
