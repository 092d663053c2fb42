"""A plain, slow implementation of Qwen2ForCausalLM: whole sequences, no
cache, one function per part, torch on the CPU.  It shares no code with the
package: it reads the model folder with the ``safetensors`` library and does
its own arithmetic, by default in float64.

It rests on the reference's formulas (cited per function; paths are those of
vjsingh1984/inferflux).  The reference's whole model cannot be compiled or
imported here: its forward includes a header of an absent submodule
(runtime/backends/llama/llama_cpp_backend.h:19 includes llama.h) and it has no
CPU model path (runtime/backends/cpu/cpu_backend.cpp:47-54 echoes tokens), so
there is no golden output of a whole model.  What pins each formula instead:

* ``embed``, ``rms_norm``, ``rope_angles`` + ``apply_rope_half``, ``silu_mul``,
  the bias add and ``causal_gqa_attention`` (group ratios 7, 3 and 5, prompt
  portions over a longer context and single tokens) are compared with the
  reference's own kernels, compiled unmodified for sm_100a, in
  ``tests/test_reference_kernels.py``;
* every function, and ``forward`` as a whole over tiny models A, B and E, is
  compared with a second implementation written separately in C++
  (``inferflux_b200/csrc/host_reference``) in ``tests/test_host_reference.py``;
* the arrangement of a layer, the tied head and the rule by which layers get a
  window (``window_of_layer``) rest on the reading alone: the reference's leaf
  kernels do not cover the first two, and it reads none of the window keys.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


def load_folder(folder: str, dtype=torch.float64) -> (dict, Dict[str, torch.Tensor]):
    """config.json as a dict and all tensors widened to ``dtype``."""
    from safetensors import safe_open
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            tensors[name] = f.get_tensor(name).to(dtype)
    return cfg, tensors


def embed(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """out[t, :] = E[id_t, :], no scale.
    runtime/backends/cuda/native/cuda_kernels.cu:599-614"""
    return table[torch.tensor(list(ids), dtype=torch.long)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w, the weight after the scale.
    runtime/backends/cuda/native/cuda_kernels.cu:469-501"""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * weight


def rope_angles(positions: torch.Tensor, rotary_dim: int, theta: float, dtype) -> (torch.Tensor, torch.Tensor):
    """f_i = 1 / theta^(2i/d), a = pos * f_i for i in [0, d/2).
    runtime/backends/cuda/native/cuda_kernels.cu:92-97"""
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float64), 2.0 * i / rotary_dim)
    a = positions.to(torch.float64)[:, None] * freq[None, :]
    return torch.cos(a).to(dtype), torch.sin(a).to(dtype)


def apply_rope_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Split-half pairs (i, i + d/2): (x0 cos - x1 sin, x0 sin + x1 cos).
    x [T, heads, d]; cos, sin [T, d/2].
    runtime/backends/cuda/native/cuda_kernels.cu:99-115 (rope_type 2)"""
    half = cos.shape[-1]
    x0, x1, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c, rest], dim=-1)


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                         window: Optional[int] = None) -> torch.Tensor:
    """q [T, nh, d], k/v [T, nkv, d] -> [T, nh, d].
    kv head = head / (nh / nkv); s = (q . k) * scale; key j visible to query i
    iff j <= i (and j > i - window); softmax; weighted sum of v.
    runtime/backends/cuda/kernels/flash_attention.cu:70-71,85,127-171"""
    t, nh, d = q.shape
    nkv = k.shape[1]
    ratio = nh // nkv
    out = torch.zeros_like(q)
    idx = torch.arange(t)
    visible = idx[None, :] <= idx[:, None]
    if window:
        visible &= idx[None, :] > idx[:, None] - window
    for h in range(nh):
        kh = h // ratio
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """a = g / (1 + exp(-g)) * u.  runtime/backends/cuda/native/cuda_kernels.cu:137-149"""
    return gate / (1.0 + torch.exp(-gate)) * up


def attention_block(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, positions: torch.Tensor,
                    nh: int, nkv: int, d: int, theta: float, window: Optional[int]) -> torch.Tensor:
    """q/k/v projections + biases, rotation of q and k, attention, output projection.
    runtime/backends/cuda/native/transformer_forward.cu:1479-1481,1514-1517,1550-1553 (projections),
    :1567-1608 (biases), :1632-1634 (rotation), :1665-1673 (attention, scale 1/sqrt(d)), :1719-1727 (o_proj)"""
    t = x.shape[0]
    q = x @ w[f"{prefix}.q_proj.weight"].T + w[f"{prefix}.q_proj.bias"]
    k = x @ w[f"{prefix}.k_proj.weight"].T + w[f"{prefix}.k_proj.bias"]
    v = x @ w[f"{prefix}.v_proj.weight"].T + w[f"{prefix}.v_proj.bias"]
    q, k, v = q.view(t, nh, d), k.view(t, nkv, d), v.view(t, nkv, d)
    cos, sin = rope_angles(positions, d, theta, x.dtype)
    q, k = apply_rope_half(q, cos, sin), apply_rope_half(k, cos, sin)
    a = causal_gqa_attention(q, k, v, 1.0 / math.sqrt(d), window)
    return a.reshape(t, nh * d) @ w[f"{prefix}.o_proj.weight"].T


def mlp_block(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down( silu(gate(x)) * up(x) ), no biases.
    runtime/backends/cuda/native/transformer_forward.cu:1877-1879,1912-1914,1981-1983,2024-2026"""
    g = x @ w[f"{prefix}.gate_proj.weight"].T
    u = x @ w[f"{prefix}.up_proj.weight"].T
    return silu_mul(g, u) @ w[f"{prefix}.down_proj.weight"].T


def window_of_layer(cfg: dict, layer: int) -> Optional[int]:
    """Layers from max_window_layers upwards attend within sliding_window when
    use_sliding_window is set (config.json keys of the architecture; the
    reference reads none of them)."""
    if cfg.get("use_sliding_window") and cfg.get("sliding_window"):
        if layer >= cfg.get("max_window_layers", cfg["num_hidden_layers"]):
            return int(cfg["sliding_window"])
    return None


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence."""
    return final_hidden(cfg, w, tokens) @ head_weight(cfg, w).T


def head_weight(cfg: dict, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    """The output head: the embedding table when there is no lm_head.weight
    (runtime/backends/cuda/native/transformer_forward.cu:2178-2183,
    runtime/backends/cuda/native/weight_map.cpp:33-37)."""
    return w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") or "lm_head.weight" not in w \
        else w["lm_head.weight"]


def final_hidden(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """The normed hidden states [T, hidden] that the output head multiplies.
    runtime/backends/cuda/native/transformer_forward.cu:1341-2202: embedding (:1376-1387); per layer
    input norm (:1413-1424), attention, residual sum + post-attention norm (:1744-1754), feed-forward,
    residual sum (:2054-2077); final norm (:2148-2151)."""
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    d = cfg.get("head_dim") or cfg["hidden_size"] // nh
    eps = cfg.get("rms_norm_eps", 1e-6)
    theta = cfg.get("rope_theta", 10000.0)
    x = embed(w["model.embed_tokens.weight"], tokens)
    positions = torch.arange(len(tokens))
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        h = rms_norm(x, w[f"{p}.input_layernorm.weight"], eps)
        x = x + attention_block(h, w, f"{p}.self_attn", positions, nh, nkv, d, theta, window_of_layer(cfg, i))
        h = rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], eps)
        x = x + mlp_block(h, w, f"{p}.mlp")
    return rms_norm(x, w["model.norm.weight"], eps)


def greedy_generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], n_new: int) -> List[int]:
    """Greedy continuation, recomputing the whole sequence for each token; the
    lowest index wins among equal maxima."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward(cfg, w, seq)[-1]
        tok = int(torch.argmax(logits))
        out.append(tok)
        seq.append(tok)
    return out


# ------------------------------------------------------------------ sampling
def apply_penalties(logits: torch.Tensor, recent: Sequence[int], rep: float, freq: float, pres: float) -> torch.Tensor:
    """For every distinct recent id: logit > 0 ? logit / rep : logit * rep; -= freq * count; -= pres.
    runtime/backends/cuda/native/gpu_sampler.cu:22-48"""
    out = logits.clone()
    counts = {}
    for t in recent:
        counts[t] = counts.get(t, 0) + 1
    for t, c in counts.items():
        v = out[t]
        v = v / rep if v > 0 else v * rep
        v = v - freq * c
        if c > 0:
            v = v - pres
        out[t] = v
    return out


def kept_probabilities(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float) -> torch.Tensor:
    """softmax(logits / T) (runtime/backends/cuda/native/gpu_sampler.cu:216-267) restricted to the top_k
    largest, then to those within min_p of the largest, then to the smallest set of the largest whose
    mass reaches top_p (:273-330); zero elsewhere, not renormalised."""
    p = torch.softmax(logits.double() / temperature, dim=-1)
    keep = torch.ones_like(p, dtype=torch.bool)
    if 0 < top_k < p.numel():
        kth = torch.sort(p, descending=True).values[top_k - 1]
        keep &= p >= kth
    if min_p > 0:
        keep &= p >= min_p * p.max()
    if 0 < top_p < 1:
        q = torch.where(keep, p, torch.zeros_like(p))
        order = torch.argsort(q, descending=True, stable=True)
        csum = torch.cumsum(q[order], 0)
        need = top_p * q.sum()
        n_keep = int((csum < need).sum()) + 1
        cut = q[order][min(n_keep, p.numel()) - 1]
        keep &= q >= cut
    return torch.where(keep, p, torch.zeros_like(p))
