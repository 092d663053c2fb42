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
        self._layer_parts: List[Dict[str, object]] = []
        for layer in spec.layers:
            arrangement = part_class("arrangement", layer.arrangement)
            parts = {role: mk(family, layer.parts[role], layer.prefix)
                     for role, family in self._roles(layer).items()}
            self._layer_parts.append(parts)
            self.blocks.append(arrangement(parts, layer.position))
        self._plan_cache()
        self._describers = self._collect_describers()

    @staticmethod
    def _roles(layer) -> Dict[str, str]:
        """role -> family for the parts a layer lists, checked against what its
        arrangement declares."""
        arrangement = part_class("arrangement", layer.arrangement)
        declared = dict(arrangement.roles)
        optional = set(getattr(arrangement, "optional_roles", ()))
        unknown = sorted(set(layer.parts) - set(declared))
        missing = sorted(set(declared) - optional - set(layer.parts))
        if unknown or missing:
            raise ValueError(f"layer '{layer.prefix}' ({layer.arrangement}): "
                             + (f"missing parts {missing}; " if missing else "")
                             + (f"parts in roles the arrangement does not have {unknown}; " if unknown else "")
                             + f"its roles are {sorted(declared)}")
        return {role: family for role, family in declared.items() if role in layer.parts}

    def _collect_describers(self):
        """One part per ``describe_key``: those asked to describe each step."""
        out = {}
        every = [self.embedding, self.final_norm, self.lm_head, *self.positions.values()]
        for parts in self._layer_parts:
            every += list(parts.values())
        for p in every:
            key = getattr(p, "describe_key", None)
            if key is not None and key not in out:
                out[key] = p
        return out

    def describe_step(self, layout, put) -> Dict[str, object]:
        return {key: p.describe_step(layout, put) for key, p in self._describers.items()}

    def step_shape(self, layout) -> tuple:
        return tuple((key, p.step_shape(layout)) for key, p in self._describers.items())

    # ------------------------------------------------------------- cache plan
    def _plan_cache(self) -> None:
        spec = self.spec
        self.kv_needs: List[KVNeed] = []
        self.runs_per_group: List[int] = []
        self.runs: List[RunInfo] = []
        self.state_needs: List[List[StateNeed]] = []
        for i, run in enumerate(spec.schedule):
            layer = spec.layers[run.layer]
            need, states = None, []
            for role, family in self._roles(layer).items():
                ps = layer.parts[role]
                cls = part_class(family, ps.kind)
                if not hasattr(cls, "kv_need"):
                    continue
                n = cls.kv_need(ps.params)
                if n is not None:
                    if need is not None:
                        raise ValueError(f"layer {run.layer}: two parts ask for a paged cache; a run has one")
                    need = n
                states += list(cls.state_needs(ps.params))
            if len({s.name for s in states}) != len(states):
                raise ValueError(f"layer {run.layer}: two state tensors of its parts have the same name")
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
            self.state_needs.append(states)
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
            for role, family in self._roles(layer).items():
                add(family, layer.parts[role], layer.prefix)
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
            for p in parts.values():
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
