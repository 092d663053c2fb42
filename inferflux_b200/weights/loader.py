"""Binding tensors of a model folder to the weights that the parts declare.

Each part lists :class:`WeightSpec` entries (full tensor name, shape, kind);
the loader reads exactly those by name and reports every fault at once:
missing tensors, tensors nobody asked for, and wrong shapes.  The reference
binds the same names (runtime/backends/cuda/native/weight_map.cpp:21-58) but
never checks a shape against the configuration and reinterprets 32-bit tensors
as 16-bit ones (weight_map.cpp:6-14); both are errors or conversions here.

Storage rule: a float tensor stored in 16 bits is kept in bfloat16 for the
bfloat16 engine and widened (exactly) for the float32 engine; a tensor stored
in 32 bits stays in 32 bits; integer tables become int32.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Dict, Iterable, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsFile, open_model_files

MATRIX, VECTOR, TABLE, IGNORED = "matrix", "vector", "table", "ignored"


@dataclass(frozen=True)
class WeightSpec:
    """One tensor that a part wants.

    kind: ``matrix`` (a float operand of a matrix product or an embedding
    table), ``vector`` (norm weights, biases: small float tensors that kernels
    read as float32), ``table`` (integers), ``ignored`` (may be present in the
    files but is not loaded, e.g. an output head that is tied to the
    embedding).
    init: how the random-weights mode fills it: ``normal`` N(0, std) or
    ``one_plus_normal`` 1 + N(0, std).
    """

    name: str
    shape: Tuple[int, ...]
    kind: str = MATRIX
    optional: bool = False
    init: str = "normal"
    std: float = 0.02


class WeightsError(ValueError):
    """Raised once, listing every missing, unexpected and misshapen tensor."""

    def __init__(self, folder: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_dtype: Sequence[Tuple[str, str]] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"weights in {folder} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtype ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {dt}" for n, dt in self.wrong_dtype))
        super().__init__("\n".join(lines))


def storage_dtype(stored: torch.dtype, kind: str, engine_dtype: torch.dtype) -> torch.dtype:
    """The dtype a loaded tensor is kept in (see the module's storage rule)."""
    if kind == TABLE:
        return torch.int32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    if engine_dtype == torch.float32:
        return torch.float32
    return torch.bfloat16


def load_weights(folder: str, specs: Iterable[WeightSpec], engine_dtype: torch.dtype,
                 device: str) -> Dict[str, torch.Tensor]:
    """Read the tensors named by ``specs`` from ``folder`` onto ``device``."""
    specs = list(specs)
    files = open_model_files(folder)
    try:
        where: Dict[str, SafetensorsFile] = {}
        for f in files:
            for n in f.names():
                where.setdefault(n, f)     # the first definition of a name wins
        wanted = {s.name: s for s in specs}
        missing = [s.name for s in specs
                   if s.name not in where and not s.optional and s.kind != IGNORED]
        unexpected = sorted(n for n in where if n not in wanted)
        wrong_shape, wrong_dtype = [], []
        for s in specs:
            if s.name in where and s.kind != IGNORED:
                dtype, shape = where[s.name].info(s.name)
                if tuple(shape) != tuple(s.shape):
                    wrong_shape.append((s.name, tuple(shape), tuple(s.shape)))
                is_float = dtype.is_floating_point
                if (s.kind == TABLE) == is_float:
                    wrong_dtype.append((s.name, str(dtype)))
        if missing or unexpected or wrong_shape or wrong_dtype:
            raise WeightsError(folder, missing, unexpected, wrong_shape, wrong_dtype)
        out: Dict[str, torch.Tensor] = {}
        for s in specs:
            if s.kind == IGNORED or s.name not in where:
                continue
            t = where[s.name].tensor(s.name)
            if t.dtype == torch.float16 and engine_dtype == torch.bfloat16:
                print(f"[inferflux_b200] note: {s.name} is stored in float16; "
                      "converted to bfloat16", file=sys.stderr)
            out[s.name] = t.to(storage_dtype(t.dtype, s.kind, engine_dtype)).to(device)
        return out
    finally:
        for f in files:
            f.close()
