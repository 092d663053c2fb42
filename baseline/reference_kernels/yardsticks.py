"""Times of the reference's own attention kernels at the benchmark's shapes.

The reference's server cannot be built offline, so ``bench.py --impl reference``
has no end-to-end number.  What can be run of the reference are its leaf
kernels; the two that its dense Qwen2.5-7B path launches for attention
(group ratio 7 is none of 2, 4, 8, so runtime/backends/cuda/kernels/flash_attention.cu:432-447
falls to ``FlashAttention2TypedKernel`` and :1203-1221 to ``FlashDecodeMultiSeq``) are timed here on the dense
``[tokens, kv_heads * head_dim]`` layout they read, with CUDA events around
eager launches (each launch runs for milliseconds, so host launch cost does not
count).  Its matrix products are ``cublasGemmEx`` calls
(runtime/backends/cuda/native/cublas_gemm.cpp:84-102): the library, not the
reference's code, so they are not timed as the reference's.
"""
from __future__ import annotations

import ctypes
import math
from typing import Dict

import torch

from . import load


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _time(fn, reps: int) -> float:
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    ev[0].record()
    for _ in range(reps):
        fn()
    ev[1].record()
    torch.cuda.synchronize()
    return ev[0].elapsed_time(ev[1]) / reps


def measure(n_heads: int = 28, n_kv_heads: int = 4, head_dim: int = 128, prompt: int = 2048, context: int = 4096,
            batches=(1, 8, 64)) -> Dict[str, dict]:
    """One layer's attention: a prompt of ``prompt`` tokens, and single tokens
    of ``batches`` requests at ``context`` cached tokens.  Milliseconds per
    launch, with the bytes or flops the launch has to move or do."""
    lib = load()
    dev, bf = "cuda:0", torch.bfloat16
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    scale = ctypes.c_float(1.0 / math.sqrt(head_dim))
    kvw = n_kv_heads * head_dim
    out: Dict[str, dict] = {}
    q = torch.randn((prompt, n_heads * head_dim), device=dev, dtype=bf)
    k = torch.randn((prompt, kvw), device=dev, dtype=bf)
    v = torch.randn((prompt, kvw), device=dev, dtype=bf)
    o = torch.empty_like(q)

    def prefill():
        rc = lib.ref_flash_attention2(_p(q), _p(k), _p(v), _p(o), 1, prompt, prompt, n_heads, n_kv_heads, head_dim,
                                      scale, 1, stream)
        assert rc == 0, rc
    ms = _time(prefill, 3)
    flops = 2 * 2 * n_heads * head_dim * (prompt * (prompt + 1) // 2)
    out[f"FlashAttention2Typed_prompt{prompt}"] = {"ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 2)}
    for b in batches:
        qd = torch.randn((b, n_heads * head_dim), device=dev, dtype=bf)
        od = torch.empty_like(qd)
        ks = [torch.randn((context, kvw), device=dev, dtype=bf) for _ in range(b)]
        vs = [torch.randn((context, kvw), device=dev, dtype=bf) for _ in range(b)]
        kp = torch.tensor([t.data_ptr() for t in ks], dtype=torch.int64, device=dev)
        vp = torch.tensor([t.data_ptr() for t in vs], dtype=torch.int64, device=dev)
        lens = torch.full((b,), context, dtype=torch.int32, device=dev)

        def decode():
            rc = lib.ref_flash_decode_multi_seq(_p(qd), _p(kp), _p(vp), _p(od), _p(lens), b, n_heads, n_kv_heads,
                                                head_dim, scale, stream)
            assert rc == 0, rc
        ms = _time(decode, 5)
        nbytes = 2 * b * context * kvw * 2
        out[f"FlashDecodeMultiSeq_batch{b}_context{context}"] = {"ms": round(ms, 4),
                                                                 "gbs": round(nbytes / ms / 1e6, 1)}
        del ks, vs
    return out
