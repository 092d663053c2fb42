"""Random weights from a configuration and a seed.

``random_tensors`` fills every tensor the model's parts declare: matrices and
biases N(0, std), norm weights 1 + N(0, std) (std 0.02 unless the part says
otherwise).  Each tensor has a generator of its own, seeded from (seed, tensor
name), so a tensor's values do not depend on which others exist.
``write_random_model`` stores them as a model folder (``config.json`` +
``model.safetensors``) that loads like any other.  The reference has no such
mode.
"""
from __future__ import annotations

import os
import zlib
from typing import Dict, Iterable

import torch

from .loader import IGNORED, TABLE, VECTOR, WeightSpec
from .safetensors_io import write_safetensors


def _seed_for(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF


def random_tensors(specs: Iterable[WeightSpec], seed: int, dtype: torch.dtype = torch.bfloat16,
                   vector_dtype: torch.dtype = None, device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Tensors for ``specs``; ``dtype`` is how matrices are stored,
    ``vector_dtype`` how norm weights and biases are (default: ``dtype``)."""
    out: Dict[str, torch.Tensor] = {}
    for s in specs:
        if s.kind == IGNORED:
            continue
        gen = torch.Generator(device=device)
        gen.manual_seed(_seed_for(seed, s.name))
        if s.kind == TABLE:
            out[s.name] = torch.zeros(s.shape, dtype=torch.int32, device=device)
            continue
        t = torch.randn(s.shape, generator=gen, dtype=torch.float32, device=device) * s.std
        if s.init == "one_plus_normal":
            t += 1.0
        store = (vector_dtype or dtype) if s.kind == VECTOR else dtype
        out[s.name] = t.to(store)
    return out


def random_tensors_as_loaded(specs: Iterable[WeightSpec], seed: int, engine_dtype: torch.dtype,
                             device: str) -> Dict[str, torch.Tensor]:
    """The tensors an engine of ``engine_dtype`` would hold after loading the
    folder that :func:`write_random_model` writes for the same seed (bfloat16
    storage, drawn on the CPU), without writing it: the command line's
    ``--random CONFIG.json`` gives the same model as ``inferctl random``
    followed by ``--model``."""
    from .loader import storage_dtype
    specs = list(specs)
    kinds = {s.name: s.kind for s in specs}
    stored = random_tensors(specs, seed, torch.bfloat16, None, "cpu")
    return {n: t.to(storage_dtype(t.dtype, kinds[n], engine_dtype)).to(device) for n, t in stored.items()}


def write_random_model(folder: str, config, seed: int, dtype: torch.dtype = torch.bfloat16,
                       vector_dtype: torch.dtype = None) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed
    model configuration) with weights from ``seed``."""
    from ..config.registry import build_spec
    from ..engine.model import Model
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    specs = Model(build_spec(config), torch.float32, "cpu").weight_specs()
    tensors = random_tensors(specs, seed, dtype, vector_dtype, "cpu")
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return folder
