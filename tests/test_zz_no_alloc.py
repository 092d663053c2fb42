"""ifx_sample_static, the sampling entry point for callers that cannot allocate
device memory (a host with a fixed memory budget, a plugin inside another
engine's pool): it keeps its scratch in a device array inside the library, so
the caller passes only inputs and outputs.  Called here through its exported C
symbol, twice in a row, and compared with the regular entry point, which gets
its scratch from the caller.  Sizes beyond the built-in scratch are refused.

The file is named so that pytest collects it last."""
from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call_static(lib, logits, temperature, top_k, top_p, min_p, seeds, counters, out):
    fn = lib.ifx_sample_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong] + [ctypes.c_void_p] * 7 + [ctypes.c_int, ctypes.c_int,
                                                                                  ctypes.c_void_p]
    r, v = logits.shape
    return fn(logits.data_ptr(), logits.stride(0), temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(),
              min_p.data_ptr(), seeds.data_ptr(), counters.data_ptr(), out.data_ptr(), r, v,
              torch.cuda.current_stream().cuda_stream)


def test_static_sampler_matches_the_regular_one_twice():
    from inferflux_b200.kernels import ops
    from inferflux_b200.kernels.build import library
    lib = library()
    lib.ifx_sample_static_message.restype = ctypes.c_char_p
    lib.ifx_sample_static_message.argtypes = [ctypes.c_int]
    f = lambda x, dt: torch.tensor(x, dtype=dt, device=DEV)
    for call, (rows, vocab, seed) in enumerate([(8, 152064, 5), (5, 1000, 6)]):   # the second call sees the first's leftovers
        g = torch.Generator().manual_seed(seed)
        logits = (torch.randn((rows, vocab), generator=g) * 3.0).to(DEV)
        temperature = f([0.8, 1.3, 0.0, 1.0, 0.5, 2.0, 0.0, 1.1][:rows], torch.float32)
        top_k = f([0, 40, 0, 5, 0, 0, 7, 1000][:rows], torch.int32)
        top_p = f([1.0, 0.9, 1.0, 0.5, 0.95, 1.0, 1.0, 0.8][:rows], torch.float32)
        min_p = f([0.0, 0.0, 0.0, 0.02, 0.0, 0.1, 0.0, 0.0][:rows], torch.float32)
        seeds = f([11 + i for i in range(rows)], torch.int64)
        counters = f([3 * i + call for i in range(rows)], torch.int64)
        want = torch.empty(rows, dtype=torch.int32, device=DEV)
        ops.sample(logits.clone(), torch.empty(rows * vocab, dtype=torch.float32, device=DEV), temperature, top_k,
                   top_p, min_p, seeds, counters, want)
        got = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
        rc = _call_static(lib, logits, temperature, top_k, top_p, min_p, seeds, counters, got)
        assert rc == 0, lib.ifx_sample_static_message(rc)
        torch.cuda.synchronize()
        assert got.tolist() == want.tolist(), f"call {call}"


def test_static_calls_back_to_back_on_one_stream():
    """Three calls queued on one stream with no synchronisation between them,
    of different sizes (so each finds the leftovers of the one before in the
    shared array), one of them reading rows that are further apart than they
    are long.  Calls on one stream run in order, which is the rule of use; each
    must still give what the regular entry point gives for its input."""
    from inferflux_b200.kernels import ops
    from inferflux_b200.kernels.build import library
    lib = library()
    f = lambda x, dt: torch.tensor(x, dtype=dt, device=DEV)
    cases = []
    for call, (rows, vocab, stride) in enumerate([(8, 50000, 50000), (3, 777, 1024), (6, 152064, 152064)]):
        g = torch.Generator().manual_seed(40 + call)
        wide = (torch.randn((rows, stride), generator=g) * 3.0).to(DEV)
        logits = wide[:, :vocab]                                   # row_stride > vocab in the second case
        temperature = f([0.9, 1.2, 0.7, 1.0, 0.0, 1.5, 0.6, 1.1][:rows], torch.float32)
        top_k = f([0, 50, 0, 8, 0, 0, 3, 400][:rows], torch.int32)
        top_p = f([1.0, 0.9, 0.8, 1.0, 1.0, 0.95, 1.0, 0.7][:rows], torch.float32)
        min_p = f([0.0, 0.0, 0.0, 0.05, 0.0, 0.0, 0.0, 0.01][:rows], torch.float32)
        seeds = f([70 + i for i in range(rows)], torch.int64)
        counters = f([5 * i + call for i in range(rows)], torch.int64)
        want = torch.empty(rows, dtype=torch.int32, device=DEV)
        ops.sample(logits.contiguous(), torch.empty(rows * vocab, dtype=torch.float32, device=DEV), temperature,
                   top_k, top_p, min_p, seeds, counters, want)
        got = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
        cases.append((logits, temperature, top_k, top_p, min_p, seeds, counters, got, want))
    torch.cuda.synchronize()
    for c in cases:                                               # queued one behind the other
        assert _call_static(lib, *c[:8]) == 0
    torch.cuda.synchronize()
    for i, c in enumerate(cases):
        assert c[7].tolist() == c[8].tolist(), f"call {i}"


def test_static_sampler_refuses_what_does_not_fit():
    from inferflux_b200.kernels.build import library
    lib = library()
    lib.ifx_sample_static_message.restype = ctypes.c_char_p
    lib.ifx_sample_static_message.argtypes = [ctypes.c_int]
    f = lambda x, dt: torch.tensor(x, dtype=dt, device=DEV)
    for rows, vocab in ((9, 100), (1, 262145)):
        logits = torch.zeros((rows, vocab), device=DEV)
        out = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
        z = lambda dt: torch.zeros(rows, dtype=dt, device=DEV)
        rc = _call_static(lib, logits, z(torch.float32), z(torch.int32), z(torch.float32), z(torch.float32),
                          z(torch.int64), z(torch.int64), out)
        assert rc == 100003
        assert b"beyond the built-in scratch" in lib.ifx_sample_static_message(rc)
        torch.cuda.synchronize()
        assert out.tolist() == [-1] * rows      # nothing was launched
