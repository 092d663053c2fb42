"""The host-side float32 reference of the model's operations
(``csrc/host_reference/host_reference.cpp``: plain C++ loops, no CUDA), built
with the system's C++ compiler into a small shared library of its own and
called through ctypes.  Only tests use it: the engine has no CPU path and never
loads this library.

Every function takes CPU tensors (float32 unless said otherwise, contiguous)
and has the signature of the matching wrapper in :mod:`inferflux_b200.kernels.ops`
as far as that makes sense on the host.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import tempfile
from typing import Optional, Sequence

import torch

SRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc", "host_reference",
                                    "host_reference.cpp"))
LIB_NAME = "libinferflux_b200_host_reference.so"
_lib: Optional[ctypes.CDLL] = None


class HostReferenceError(RuntimeError):
    pass


def build() -> str:
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise HostReferenceError("no C++ compiler (g++ / c++ / $CXX) was found")
    with open(SRC, "rb") as f:
        digest = hashlib.sha256(f.read()).hexdigest()[:16]
    out_dir = os.path.join(os.path.dirname(SRC), "..", "_build")
    try:
        os.makedirs(out_dir, exist_ok=True)
        probe = os.path.join(out_dir, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
    except OSError:
        out_dir = os.path.join(tempfile.gettempdir(), f"inferflux_b200_build_{os.getuid()}")
        os.makedirs(out_dir, exist_ok=True)
    lib = os.path.join(out_dir, LIB_NAME)
    stamp = lib + ".stamp"
    if os.path.isfile(lib) and os.path.isfile(stamp) and open(stamp).read().strip() == digest:
        return lib
    # no -ffast-math: the order of every sum is the one written in the source
    r = subprocess.run([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-o", lib, SRC],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise HostReferenceError(f"{cxx} failed on host_reference.cpp:\n{r.stdout}\n{r.stderr}")
    with open(stamp, "w") as f:
        f.write(digest)
    return lib


def library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.hr_uniform01.restype = ctypes.c_double
        _lib.hr_uniform01.argtypes = [ctypes.c_uint64, ctypes.c_uint64]
        _lib.hr_inverse_cdf.restype = ctypes.c_int
        _lib.hr_inverse_cdf.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_double]
        _lib.hr_model_step.restype = ctypes.c_int
    return _lib


def _f32(t: torch.Tensor) -> torch.Tensor:
    if t.device.type != "cpu" or t.dtype != torch.float32 or not t.is_contiguous():
        raise HostReferenceError("the host reference takes contiguous float32 CPU tensors")
    return t


def _i32(t: torch.Tensor) -> torch.Tensor:
    if t.device.type != "cpu" or t.dtype != torch.int32 or not t.is_contiguous():
        raise HostReferenceError("the host reference takes contiguous int32 CPU tensors for indices")
    return t


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_F, _L = ctypes.c_float, ctypes.c_long


def embed_gather(table, ids, out):
    library().hr_embed_gather(_p(_f32(table)), _p(_i32(ids)), _p(_f32(out)), ids.numel(), table.shape[1])
    return out


def add_rmsnorm(residual, delta, weight, eps, out, rows=None, n_partials=1):
    n, hidden = residual.shape
    library().hr_add_rmsnorm(_p(_f32(residual)), _p(None if delta is None else _f32(delta)), n_partials,
                             _p(_f32(weight)), _F(eps), _p(None if out is None else _f32(out)),
                             _p(None if rows is None else _i32(rows)), 0 if rows is None else rows.numel(), n, hidden)
    return out


def swiglu(gate_up, out):
    library().hr_swiglu(_p(_f32(gate_up)), _p(_f32(out)), out.shape[0], out.shape[1])
    return out


def gemm(a, w, bias, out):
    library().hr_gemm(_p(_f32(a)), _p(_f32(w)), _p(None if bias is None else _f32(bias)), _p(_f32(out)),
                      a.shape[0], w.shape[0], a.shape[1])
    return out


def rope_table(positions, inv_freq, cos, sin):
    if inv_freq.dtype != torch.float64 or not inv_freq.is_contiguous():
        raise HostReferenceError("inv_freq is float64")
    library().hr_rope_table(_p(_i32(positions)), _p(inv_freq), _p(_f32(cos)), _p(_f32(sin)), positions.numel(),
                            inv_freq.numel())


def qkv_rope_kv_write(qkv, bias, cos, sin, slot_map, k_layer, v_layer, page_stride, page_size, n_heads, n_kv, head_dim):
    """k_layer / v_layer: the views [n_kv, page_size, head_dim] of page 0 of one run (as the kernel wrapper gets them)."""
    library().hr_qkv_rope_kv_write(
        _p(_f32(qkv)), _p(None if bias is None else _f32(bias)), _p(_f32(cos)), _p(_f32(sin)), cos.shape[1],
        _p(None if slot_map is None else _i32(slot_map)), _p(k_layer), _p(v_layer), _L(page_stride), page_size,
        qkv.shape[0], n_heads, n_kv, head_dim)


def attention_paged(q, q_stride, out, k_layer, v_layer, page_stride, page_size, block_tables, entry_q_start,
                    entry_q_len, entry_ctx_start, n_heads, n_kv, head_dim, scale, window):
    library().hr_attention_paged(
        _p(_f32(q)), _L(q_stride), _p(_f32(out)), _L(out.stride(0)), _p(k_layer), _p(v_layer), _L(page_stride),
        page_size, _p(_i32(block_tables)), block_tables.shape[1], _p(_i32(entry_q_start)), _p(_i32(entry_q_len)),
        _p(_i32(entry_ctx_start)), entry_q_start.numel(), n_heads, n_kv, head_dim, _F(scale), int(window or 0))
    return out


def argmax(logits, out):
    if logits.stride(1) != 1 or logits.dtype != torch.float32:
        raise HostReferenceError("argmax: float32 rows")
    library().hr_argmax(_p(logits), _L(logits.stride(0)), _p(_i32(out)), logits.shape[0], logits.shape[1])
    return out


def apply_penalties(logits, recent_ids, recent_counts, n_recent, rep, freq, pres):
    library().hr_apply_penalties(_p(_f32(logits)), _p(_i32(recent_ids)), _p(_i32(recent_counts)), _p(_i32(n_recent)),
                                 recent_ids.shape[1], _p(_f32(rep)), _p(_f32(freq)), _p(_f32(pres)), logits.shape[0],
                                 logits.shape[1])


def kept_probabilities(logits, temperature, top_k, top_p, min_p) -> torch.Tensor:
    probs = torch.empty(logits.numel(), dtype=torch.float64)
    library().hr_kept_probabilities(_p(_f32(logits)), logits.numel(), _F(temperature), int(top_k), _F(top_p),
                                    _F(min_p), _p(probs))
    return probs


def uniform01(seed: int, counter: int) -> float:
    return float(library().hr_uniform01(seed & (2 ** 64 - 1), counter & (2 ** 64 - 1)))


def inverse_cdf(probs: torch.Tensor, u: float) -> int:
    return int(library().hr_inverse_cdf(_p(probs), probs.numel(), u))


# ---------------------------------------------------------------- whole model
class _Layer(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("input_norm", "wq", "wk", "wv", "bq", "bk", "bv", "wo", "post_norm",
                                               "w_gate", "w_up", "w_down")] + [("window", ctypes.c_int),
                                                                                ("pad", ctypes.c_int)]


class _Model(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("hidden", "n_heads", "n_kv", "head_dim", "inter", "vocab", "n_layers",
                                            "pad")] + [("eps", ctypes.c_float), ("pad2", ctypes.c_float),
                                                       ("theta", ctypes.c_double), ("embed", ctypes.c_void_p),
                                                       ("final_norm", ctypes.c_void_p), ("lm_head", ctypes.c_void_p),
                                                       ("layers", ctypes.POINTER(_Layer))]


class HostModel:
    """The whole model on the host over a paged cache of its own.

    ``weights``: float32 CPU tensors by their names in the model folder;
    ``windows``: per layer, 0 or None = every key.  ``step`` runs entries
    ``(block table, cached tokens, new tokens, wanted places)`` as one batch."""

    def __init__(self, hidden, n_heads, n_kv, head_dim, inter, vocab, n_layers, eps, theta, tied, weights,
                 windows: Sequence[Optional[int]], num_pages: int, page_size: int):
        self._keep = {k: _f32(v.contiguous()) for k, v in weights.items()}
        w = self._keep
        layers = (_Layer * n_layers)()
        for i in range(n_layers):
            p = f"model.layers.{i}."
            g = lambda name: w[p + name].data_ptr() if p + name in w else 0
            layers[i] = _Layer(g("input_layernorm.weight"), g("self_attn.q_proj.weight"), g("self_attn.k_proj.weight"),
                               g("self_attn.v_proj.weight"), g("self_attn.q_proj.bias"), g("self_attn.k_proj.bias"),
                               g("self_attn.v_proj.bias"), g("self_attn.o_proj.weight"),
                               g("post_attention_layernorm.weight"), g("mlp.gate_proj.weight"),
                               g("mlp.up_proj.weight"), g("mlp.down_proj.weight"), int(windows[i] or 0), 0)
        self._layers = layers
        head = w["model.embed_tokens.weight"] if tied or "lm_head.weight" not in w else w["lm_head.weight"]
        self._model = _Model(hidden, n_heads, n_kv, head_dim, inter, vocab, n_layers, 0, eps, 0.0, theta,
                             w["model.embed_tokens.weight"].data_ptr(), w["model.norm.weight"].data_ptr(),
                             head.data_ptr(), layers)
        self.vocab, self.page_size = vocab, page_size
        self.pool = torch.zeros((num_pages, n_layers, 2, n_kv, page_size, head_dim), dtype=torch.float32)

    def step(self, entries) -> torch.Tensor:
        tokens, q_start, q_len, ctx, want = [], [], [], [], []
        width = max(len(e[0]) for e in entries)
        tables = torch.full((len(entries), width), -1, dtype=torch.int32)
        for i, (table, cached, new, places) in enumerate(entries):
            tables[i, :len(table)] = torch.tensor(table, dtype=torch.int32)
            q_start.append(len(tokens)), q_len.append(len(new)), ctx.append(cached)
            want += [len(tokens) + p for p in places]
            tokens += list(new)
        it = lambda v: torch.tensor(v, dtype=torch.int32)
        logits = torch.empty((len(want), self.vocab), dtype=torch.float32)
        t, qs, ql, cs, wr = it(tokens), it(q_start), it(q_len), it(ctx), it(want)
        rc = library().hr_model_step(ctypes.byref(self._model), _p(self.pool), self.page_size, _p(t), len(tokens),
                                     _p(qs), _p(ql), _p(cs), len(entries), _p(tables), width, _p(wr), len(want),
                                     _p(logits))
        if rc != 0:
            raise HostReferenceError(f"hr_model_step returned {rc}: a position has no page")
        return logits
