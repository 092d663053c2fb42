"""A model assembled from a :class:`~inferflux_b200.config.spec.ModelSpec`.

The model builds each layer's parts from the registries, works out which runs
share a cache group, collects the weights the parts declare, and runs a step:
embedding, the runs in schedule order, final norm and output head at the
wanted rows.  (Reference: the same sequence is hard-coded in
runtime/backends/cuda/native/transformer_forward.cu:1341-2202 for a whole
prompt and :2261-3358 for a decode batch.)
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.registry import part_class
from ..config.spec import ModelSpec
from ..parts.base import KVNeed, RunInfo, StateNeed
from ..weights.loader import WeightSpec, load_weights


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: str):
        spec.validate()
        self.spec = spec
        self.dtype = dtype
        self.device = device
        mk = lambda family, ps, prefix="": part_class(family, ps.kind)(ps.params, prefix, dtype, device)
        self.embedding = mk("embedding", spec.embedding)
        self.final_norm = mk("norm", spec.final_norm)
        self.lm_head = mk("lm_head", spec.lm_head)
        self.positions = {name: mk("position", ps) for name, ps in spec.positions.items()}
        self.blocks = []
        self._layer_parts = []
        for layer in spec.layers:
            mixer = mk("mixer", layer.mixer, layer.prefix)
            mixer_norm = mk("norm", layer.mixer_norm, layer.prefix)
            ffn = mk("feed_forward", layer.feed_forward, layer.prefix)
            ffn_norm = mk("norm", layer.feed_forward_norm, layer.prefix)
            self._layer_parts.append((mixer, mixer_norm, ffn, ffn_norm))
            arrangement = part_class("arrangement", layer.arrangement)
            self.blocks.append(arrangement(mixer, mixer_norm, ffn, ffn_norm, layer.position))
        self._plan_cache()

    # ------------------------------------------------------------- cache plan
    def _plan_cache(self) -> None:
        spec = self.spec
        self.kv_needs: List[KVNeed] = []
        self.runs_per_group: List[int] = []
        self.runs: List[RunInfo] = []
        self.state_needs: List[List[StateNeed]] = []
        for i, run in enumerate(spec.schedule):
            layer = spec.layers[run.layer]
            cls = part_class("mixer", layer.mixer.kind)
            need = cls.kv_need(layer.mixer.params)
            info = RunInfo(run_index=i)
            if run.cache_of is not None:
                if need is not None:
                    raise ValueError(f"schedule[{i}]: layer {run.layer} writes keys and values of its own "
                                     f"but is told to read the cache of run {run.cache_of}")
                src = self.runs[run.cache_of]
                if src.kv_group is None:
                    raise ValueError(f"schedule[{i}]: run {run.cache_of} has no paged cache to read")
                info.kv_group, info.kv_index, info.writes_kv = src.kv_group, src.kv_index, False
            elif need is not None:
                if need not in self.kv_needs:
                    self.kv_needs.append(need)
                    self.runs_per_group.append(0)
                g = self.kv_needs.index(need)
                info.kv_group, info.kv_index = g, self.runs_per_group[g]
                self.runs_per_group[g] += 1
            self.state_needs.append(list(cls.state_needs(layer.mixer.params)))
            self.runs.append(info)

    def attach_states(self, storage) -> None:
        for info in self.runs:
            info.states = storage.of_run(info.run_index)

    # ---------------------------------------------------------------- weights
    def weight_specs(self) -> List[WeightSpec]:
        spec = self.spec
        out: Dict[str, WeightSpec] = {}

        def add(family, ps, prefix=""):
            for w in part_class(family, ps.kind).weight_specs(ps.params, prefix):
                prev = out.get(w.name)
                if prev is not None and prev.kind == "ignored":
                    continue
                if prev is None or w.kind != "ignored":
                    out[w.name] = w
        add("embedding", spec.embedding)
        for layer in spec.layers:
            add("mixer", layer.mixer, layer.prefix)
            add("norm", layer.mixer_norm, layer.prefix)
            add("feed_forward", layer.feed_forward, layer.prefix)
            add("norm", layer.feed_forward_norm, layer.prefix)
        add("norm", spec.final_norm)
        add("lm_head", spec.lm_head)
        for ps in spec.positions.values():               # a position encoding may have weights of its own
            add("position", ps)
        return list(out.values())

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Hand the loaded tensors to the parts (which may fuse and drop them)."""
        self.weight_bytes = sum(t.numel() * t.element_size() for t in tensors.values())
        self.embedding.load(tensors)
        self.lm_head.load(tensors)
        self.final_norm.load(tensors)
        for parts in self._layer_parts:
            for p in parts:
                p.load(tensors)
        for p in self.positions.values():
            p.load(tensors)

    def load_folder(self, folder: str) -> None:
        self.load(load_weights(folder, self.weight_specs(), self.dtype, self.device))

    # ------------------------------------------------------------------- step
    def forward(self, ctx) -> torch.Tensor:
        """Run the step's tokens through every run; float32 logits [n_want, vocab]."""
        for name, pos in self.positions.items():
            ctx.position_tables[name] = pos.prepare(ctx)
        residual = self.embedding.forward(ctx.token_ids)
        delta = None
        for info in self.runs:
            delta = self.blocks[self.spec.schedule[info.run_index].layer].forward(residual, delta, ctx, info)
        if ctx.n_want == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        x = self.final_norm.forward(residual, delta, rows=ctx.want_rows)
        return self.lm_head.forward(x)
