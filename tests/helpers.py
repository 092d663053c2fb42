"""Shared test helpers: the tiny configurations, model folders in temporary
directories, a driver for bin/trace_run, tolerances."""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Two tiny configurations that differ in every size and option.
TINY_A = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=64, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=176, vocab_size=512,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=256,
              use_sliding_window=False, hidden_act="silu", torch_dtype="bfloat16")
TINY_B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=96, num_hidden_layers=3,
              num_attention_heads=3, num_key_value_heads=1, head_dim=32, intermediate_size=256, vocab_size=1000,
              rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=512,
              use_sliding_window=False, hidden_act="silu", torch_dtype="bfloat16")
# head_dim * heads != hidden, 5 query heads per kv head, an odd vocabulary
TINY_C = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=80, num_hidden_layers=2,
              num_attention_heads=10, num_key_value_heads=2, head_dim=48, intermediate_size=136, vocab_size=777,
              rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=384,
              use_sliding_window=False, hidden_act="silu", torch_dtype="bfloat16")
# head_dim 64: the size the tensor-core attention kernels take; 3 query heads per kv head, a window
TINY_D = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_size=120, num_hidden_layers=2,
              num_attention_heads=6, num_key_value_heads=2, head_dim=64, intermediate_size=200, vocab_size=600,
              rope_theta=200000.0, rms_norm_eps=2e-6, tie_word_embeddings=True, max_position_embeddings=400,
              use_sliding_window=True, sliding_window=70, max_window_layers=1, hidden_act="silu",
              torch_dtype="bfloat16")
# B's sizes with a window of 40 keys on all layers but the first: two cache groups, pages given back behind the window
TINY_E = dict(TINY_B, use_sliding_window=True, sliding_window=40, max_window_layers=1)
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}

# Largest |engine - plain| allowed, as a fraction of the largest |plain logit|.
# float32: a few hundred float32 roundings; bfloat16: 8-bit mantissas through every layer.
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def make_model_folder(cfg: dict, seed: int, folder: Optional[str] = None, sharpen: float = 6.0,
                      vector_dtype=None) -> str:
    """Write a random model folder.  ``sharpen`` multiplies the q and k
    projection weights so that attention is peaked: with N(0, 0.02) weights it
    is nearly uniform and one wrong key among many would hide below the
    bfloat16 tolerance."""
    from inferflux_b200.config import Qwen2Config
    from inferflux_b200.config.registry import build_spec
    from inferflux_b200.engine.model import Model
    from inferflux_b200.weights.random_init import random_tensors
    from inferflux_b200.weights.safetensors_io import write_safetensors
    folder = folder or tempfile.mkdtemp(prefix="ifx_model_")
    config = Qwen2Config.from_dict(cfg)
    config.save(folder)
    specs = Model(build_spec(config), torch.float32, "cpu").weight_specs()
    tensors = random_tensors(specs, seed, torch.bfloat16, vector_dtype, "cpu")
    if sharpen != 1.0:
        for name in tensors:
            if name.endswith(("q_proj.weight", "k_proj.weight")):
                tensors[name] = (tensors[name].float() * sharpen).to(tensors[name].dtype)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder


def random_tokens(vocab: int, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class TraceProcess:
    """A running bin/trace_run: send steps, wait for ``done``, read logits."""

    def __init__(self, model_dir: Optional[str], dtype: str, max_tokens: int, extra: Sequence[str] = ()):
        self.out = tempfile.mkdtemp(prefix="ifx_trace_")
        self.step_no = 0
        cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), *(["--model", model_dir] if model_dir else []),
               "--dtype", dtype, "--out", self.out, "--max-tokens", str(max_tokens), *extra]
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)

    def step(self, entries: Sequence[dict], end: Sequence[str] = ()) -> Optional[np.ndarray]:
        """entries: dicts with id, tokens, want.  Returns [wanted, vocab] or None."""
        n = self.step_no
        self.step_no += 1
        self.proc.stdin.write(json.dumps({"step": n, "entries": list(entries), "end": list(end)}) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.strip() != f"done {n}":
            rc = self.proc.poll()
            raise RuntimeError(f"trace_run answered {line!r} to step {n} (exit code {rc})")
        wanted = sum(len(e.get("want", [])) for e in entries)
        if not wanted:
            return None
        arr = np.fromfile(os.path.join(self.out, f"{n}.f32"), dtype="<f4")
        return arr.reshape(wanted, -1)

    def stats(self) -> dict:
        """The counters of the cache pools and of the step function."""
        self.proc.stdin.write(json.dumps({"stats": True}) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if not line.startswith("stats "):
            raise RuntimeError(f"trace_run answered {line!r} to a request for its counters")
        return json.loads(line[len("stats "):])

    def close(self) -> int:
        self.proc.stdin.close()
        rc = self.proc.wait(timeout=120)
        return rc


def rel_err(got, ref) -> float:
    got = torch.as_tensor(np.asarray(got), dtype=torch.float64)
    ref = torch.as_tensor(np.asarray(ref), dtype=torch.float64)
    return float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
