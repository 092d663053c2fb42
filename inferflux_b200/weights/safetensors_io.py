"""Reading and writing the safetensors container.

Format (as the reference parses it,
runtime/backends/cuda/native/safetensors_parser.cpp:144-177 header,
:179-259 per-tensor metadata, :261-303 data): an unsigned 64-bit little-endian
header length, a JSON object that maps each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the
end of the header; keys that start with ``__`` are metadata and skipped), then
the raw little-endian tensor bytes.  The reference only warns when a tensor's
byte size disagrees with its shape (safetensors_parser.cpp:292-299); here that
is an error.

Sharded models carry ``model.safetensors.index.json`` whose ``weight_map``
maps tensor names to shard files (inferflux_cuda_executor.cpp:356-392).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, List, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16,
    "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
    "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are views into the mapping."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(
                f"{path}: header length {hlen} is beyond the file ({size} bytes) or the 100 MB limit")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self._data_start = 8 + hlen
        data_bytes = size - self._data_start
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, meta in header.items():
            if name.startswith("__"):
                continue
            try:
                dt, shape, (b, e) = meta["dtype"], tuple(int(s) for s in meta["shape"]), meta["data_offsets"]
            except (KeyError, TypeError, ValueError) as err:
                raise SafetensorsError(f"{path}: tensor '{name}' has a malformed entry ({err})") from err
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype '{dt}'")
            dtype = _DTYPES[dt]
            numel = 1
            for s in shape:
                numel *= s
            nbytes = numel * torch.empty((), dtype=dtype).element_size()
            if not (0 <= b <= e <= data_bytes):
                raise SafetensorsError(
                    f"{path}: tensor '{name}' data_offsets [{b}, {e}) lie outside the data ({data_bytes} bytes)")
            if e - b != nbytes:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' has {e - b} bytes but shape {list(shape)} of {dt} needs {nbytes}")
            self.entries[name] = (dtype, shape, int(b), int(e))
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self.entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that copies the named tensor out of the mapping."""
        dtype, shape, b, e = self.entries[name]
        if e == b:
            return torch.empty(shape, dtype=dtype)
        raw = np.frombuffer(self._mm, dtype=np.uint8, count=e - b, offset=self._data_start + b)
        flat = torch.from_numpy(raw.copy()).view(dtype)
        return flat.reshape(shape)

    def close(self) -> None:
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass
            self._mm = None
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Write tensors (moved to the CPU, made contiguous) in name order."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}' has dtype {t.dtype}, which safetensors cannot hold")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    pad = (8 - (8 + len(blob)) % 8) % 8   # data starts on an 8-byte boundary
    blob += b" " * pad
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)


def open_model_files(folder: str) -> List[SafetensorsFile]:
    """The shard files of a model folder: those of the index if there is one,
    else ``model.safetensors``."""
    index = os.path.join(folder, "model.safetensors.index.json")
    single = os.path.join(folder, "model.safetensors")
    if os.path.isfile(index):
        with open(index) as f:
            wm = json.load(f).get("weight_map", {})
        shards = sorted(set(wm.values()))
        if not shards:
            raise SafetensorsError(f"{index}: weight_map is empty")
        missing = [s for s in shards if not os.path.isfile(os.path.join(folder, s))]
        if missing:
            raise SafetensorsError(f"{index}: shard files are missing: {missing}")
        return [SafetensorsFile(os.path.join(folder, s)) for s in shards]
    if os.path.isfile(single):
        return [SafetensorsFile(single)]
    raise SafetensorsError(f"no safetensors files found in {folder} "
                           "(expected model.safetensors or model.safetensors.index.json)")
