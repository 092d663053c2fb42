"""Compiling the CUDA sources under ``csrc/`` for sm_100a and loading the
resulting shared library through ctypes.

The library has a plain C interface (``extern "C"``, raw pointers and a
stream), so it needs no Python or torch headers and compiles in seconds per
file.  It is built in-tree under ``csrc/_build`` at the first call and rebuilt
when a source or a flag changes; when the tree is read-only the build goes to a
per-user folder under the system's temporary directory.  There is no fallback:
if the library cannot be built or loaded, every kernel call raises.
"""
from __future__ import annotations

import concurrent.futures
import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import List, Optional

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
LIB_NAME = "libinferflux_b200_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]
# INFERFLUX_B200_TIMELINE=1 selects an instrumented build (a library of its own beside the serving one) in
# which every kernel notes the global timer when its predecessor is complete; cli/kernel_bench.py reads it.
TIMELINE = os.environ.get("INFERFLUX_B200_TIMELINE", "") not in ("", "0")
OBJ_SUFFIX = ".tl.o" if TIMELINE else ".o"
if TIMELINE:
    LIB_NAME = "libinferflux_b200_kernels_timeline.so"
    NVCC_FLAGS = NVCC_FLAGS + ["-DIFX_TIMELINE"]
# INFERFLUX_B200_NVCC_EXTRA="-DX=1 ..." adds compiler flags (kernel experiments); such a build is a library of
# its own too, named after the flags, so it never stands in for the serving one.
EXTRA = os.environ.get("INFERFLUX_B200_NVCC_EXTRA", "").split()
if EXTRA:
    tag = hashlib.sha256(" ".join(EXTRA).encode()).hexdigest()[:8]
    LIB_NAME = LIB_NAME[:-3] + f"_{tag}.so"
    OBJ_SUFFIX = f".x{tag}" + OBJ_SUFFIX
    NVCC_FLAGS = NVCC_FLAGS + EXTRA

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("nvcc was not found (PATH, $NVCC, /usr/local/cuda/bin); "
                           "the CUDA kernels cannot be built and there is no fallback")


def _sources() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _digest(paths: List[str], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    d = os.environ.get("INFERFLUX_B200_BUILD_DIR") or os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"inferflux_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[inferflux_b200 build] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, obj: str, verbose_ptxas: bool) -> str:
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj]
    if verbose_ptxas:
        cmd += ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise KernelBuildError(f"nvcc failed on {os.path.basename(src)}:\n{r.stdout}\n{r.stderr}")
    return r.stderr


def build(force: bool = False, verbose_ptxas: bool = False) -> str:
    """Compile every ``.cu`` under csrc (in parallel) and link the library.
    Returns the library's path."""
    nvcc = _nvcc()
    srcs, hdrs = _sources(), _headers()
    if not srcs:
        raise KernelBuildError(f"no CUDA sources under {CSRC}")
    out_dir = _build_dir()
    flags_key = " ".join(ARCH_FLAGS + NVCC_FLAGS)
    hdr_key = _digest(hdrs, flags_key)
    lib_path = os.path.join(out_dir, LIB_NAME)
    stamp_path = lib_path + ".stamp"
    total = _digest(srcs + hdrs, flags_key)
    if not force and os.path.isfile(lib_path) and os.path.isfile(stamp_path):
        with open(stamp_path) as f:
            if f.read().strip() == total:
                return lib_path
    todo = []
    objs = []
    for src in srcs:
        key = _digest([src], hdr_key)
        obj = os.path.join(out_dir, os.path.basename(src)[:-3] + f".{key}{OBJ_SUFFIX}")
        objs.append(obj)
        if force or not os.path.isfile(obj):
            todo.append((src, obj))
    t0 = time.time()
    if todo:
        _say(f"compiling {len(todo)} CUDA source file(s) for sm_100a into {out_dir} "
             "(first call only)")
        workers = max(1, min(len(todo), os.cpu_count() or 1))
        with concurrent.futures.ThreadPoolExecutor(workers) as pool:
            futs = {pool.submit(_compile_one, nvcc, s, o + ".tmp.o", verbose_ptxas): (s, o)
                    for s, o in todo}
            pending = set(futs)
            done_n = 0
            while pending:
                done, pending = concurrent.futures.wait(pending, timeout=10.0)
                for fu in done:
                    s, o = futs[fu]
                    log = fu.result()
                    os.replace(o + ".tmp.o", o)
                    done_n += 1
                    _say(f"  [{done_n}/{len(todo)}] {os.path.basename(s)} "
                         f"({time.time() - t0:.0f} s)")
                    if verbose_ptxas and log:
                        sys.stderr.write(log)
                if pending and not done:
                    _say(f"  still compiling, {len(pending)} file(s) left "
                         f"({time.time() - t0:.0f} s)")
    tmp_lib = lib_path + f".tmp{os.getpid()}"
    cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp_lib, *objs, "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise KernelBuildError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp_lib, lib_path)
    with open(stamp_path, "w") as f:
        f.write(total)
    # drop objects of older source versions
    keep = {os.path.basename(o) for o in objs}
    for f in os.listdir(out_dir):
        if f.endswith(OBJ_SUFFIX) and (EXTRA or ".x" not in f) and f.endswith(".tl.o") == TIMELINE and f not in keep:
            try:
                os.remove(os.path.join(out_dir, f))
            except OSError:
                pass
    if todo:
        _say(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
    return lib_path


def library() -> ctypes.CDLL:
    """The loaded kernel library (built first if needed)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = build()
            try:
                _lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from e
    return _lib


def library_path() -> str:
    return build()
