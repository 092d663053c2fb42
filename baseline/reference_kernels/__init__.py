"""The leaf CUDA kernels of vjsingh1984/inferflux, compiled unmodified for
sm_100a and callable from Python.

The reference's server and its forward pass cannot be built offline (the
forward includes ``llama.h`` of a submodule that is empty in the snapshot), but
two of its kernel files include nothing outside their own tree:
``runtime/backends/cuda/native/cuda_kernels.cu`` (embedding, norms, rotation,
bias, SiLU) and ``runtime/backends/cuda/kernels/flash_attention.cu`` (the
attention kernels that its dense path launches).  They serve two purposes here:

* an anchor for the formulas: ``tests/test_reference_kernels.py`` compares each
  of them with the plain implementation under ``tests/``;
* the kernels to beat: ``bench.py --impl reference`` times the reference's
  attention at the benchmark's shapes.

The sources are not part of this repository.  ``python -m
baseline.reference_kernels fetch <reference checkout>`` copies the files named
in :data:`SOURCE_FILES`, byte for byte, to ``baseline/_ref/inferflux_src``
(ignored by git); :func:`load` compiles them there together with ``harness.cu``
(C entry points that only forward their arguments).
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
from typing import Optional

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.normpath(os.path.join(HERE, "..", "_ref"))
SOURCE_ROOT = os.path.join(REF_DIR, "inferflux_src")
SOURCE_FILES = (
    "runtime/backends/cuda/common/dtype_traits.cuh",
    "runtime/backends/cuda/native/cuda_kernels.cu",
    "runtime/backends/cuda/native/cuda_kernels.cuh",
    "runtime/backends/cuda/kernels/flash_attention.cu",
    "runtime/backends/cuda/kernels/flash_attention.cuh",
    "runtime/backends/cuda/kernels/flash_attention_mma.cuh",
)
COMPILED = ("runtime/backends/cuda/native/cuda_kernels.cu", "runtime/backends/cuda/kernels/flash_attention.cu")
LIB_NAME = "libinferflux_reference_kernels.so"


class ReferenceUnavailable(RuntimeError):
    """The reference's sources are not here, or they did not compile."""


def fetch(checkout: str) -> str:
    """Copy the files of :data:`SOURCE_FILES` from a checkout of the reference."""
    for rel in SOURCE_FILES:
        src = os.path.join(checkout, rel)
        if not os.path.isfile(src):
            raise ReferenceUnavailable(f"{src} does not exist")
        dst = os.path.join(SOURCE_ROOT, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(src, dst)
    return SOURCE_ROOT


def source_root() -> Optional[str]:
    root = os.environ.get("INFERFLUX_REFERENCE_SRC") or SOURCE_ROOT
    if all(os.path.isfile(os.path.join(root, rel)) for rel in SOURCE_FILES):
        return root
    return None


def _build_dir() -> str:
    d = os.path.join(REF_DIR, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"inferflux_reference_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


_lib: Optional[ctypes.CDLL] = None


def build() -> str:
    """Compile the reference's two kernel files and the harness into one
    shared library (once; again when a source changes).  Returns its path."""
    root = source_root()
    if root is None:
        raise ReferenceUnavailable(
            f"the reference's kernel sources are not under {SOURCE_ROOT}; "
            "run: python -m baseline.reference_kernels fetch <reference checkout>")
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(nvcc):
        raise ReferenceUnavailable("nvcc was not found")
    srcs = [os.path.join(HERE, "harness.cu")] + [os.path.join(root, rel) for rel in COMPILED]
    h = hashlib.sha256()
    for p in srcs + [os.path.join(root, rel) for rel in SOURCE_FILES]:
        with open(p, "rb") as f:
            h.update(f.read())
    out_dir = _build_dir()
    lib = os.path.join(out_dir, LIB_NAME)
    stamp = lib + ".stamp"
    if os.path.isfile(lib) and os.path.isfile(stamp) and open(stamp).read().strip() == h.hexdigest():
        return lib
    print("[reference kernels] compiling the reference's cuda_kernels.cu and flash_attention.cu for sm_100a ...",
          file=sys.stderr, flush=True)
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
           "-shared", "-I", root, "-o", lib, *srcs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise ReferenceUnavailable(f"nvcc failed on the reference's kernels:\n{r.stdout}\n{r.stderr}")
    with open(stamp, "w") as f:
        f.write(h.hexdigest())
    return lib


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib

