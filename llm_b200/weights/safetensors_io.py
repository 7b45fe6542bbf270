"""Reader and writer of the safetensors container.

Layout: 8 bytes little-endian header length N, N bytes of JSON
(name -> {dtype, shape, data_offsets}), then the tensors' bytes.  The checks are
those of the reference's index reader (utils/safetensor_loader.h:64-95): file
shorter than 8 bytes, header larger than the file, missing dtype / shape /
data_offsets, reversed offsets, a tensor past the end, an unsupported dtype; and,
beyond it, a byte count that does not match the shape.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Dict, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# name in the file -> (torch dtype, bytes per element, numpy carrier dtype)
_DTYPES = {
    "F32": (torch.float32, 4, np.float32),
    "BF16": (torch.bfloat16, 2, np.int16),
    "F16": (torch.float16, 2, np.float16),
    "I32": (torch.int32, 4, np.int32),
    "I64": (torch.int64, 8, np.int64),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    dtype: torch.dtype
    shape: Tuple[int, ...]
    start: int   # offsets into the data section
    end: int


class SafetensorsFile:
    """An opened file: the index, and tensors as views of the mapped bytes."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open: {e}") from e
        if size < 8:
            raise SafetensorsError(f"{path}: shorter than the 8-byte header length")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.data_start = 8 + hlen
        data_len = size - self.data_start
        self.metadata = header.pop("__metadata__", None)
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            if not isinstance(info, dict):
                raise SafetensorsError(f"{path}: entry '{name}' is not an object")
            for key in ("dtype", "shape", "data_offsets"):
                if key not in info:
                    raise SafetensorsError(f"{path}: tensor '{name}' has no '{key}'")
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {info['dtype']!r}")
            offs = info["data_offsets"]
            if not (isinstance(offs, list) and len(offs) == 2 and all(isinstance(o, int) for o in offs)):
                raise SafetensorsError(f"{path}: tensor '{name}': data_offsets must be two integers")
            start, end = offs
            if start < 0 or end < start:
                raise SafetensorsError(f"{path}: tensor '{name}': reversed data_offsets {offs}")
            if end > data_len:
                raise SafetensorsError(f"{path}: tensor '{name}' ends at {end}, past the data section ({data_len})")
            shape = tuple(info["shape"])
            if not all(isinstance(s, int) and s >= 0 for s in shape):
                raise SafetensorsError(f"{path}: tensor '{name}': bad shape {info['shape']}")
            tdtype, esize, _ = _DTYPES[info["dtype"]]
            numel = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if numel * esize != end - start:
                raise SafetensorsError(
                    f"{path}: tensor '{name}': shape {list(shape)} of {info['dtype']} needs {numel * esize} "
                    f"bytes, data_offsets give {end - start}")
            self.entries[name] = TensorEntry(tdtype, shape, start, end)
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self):
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (read-only memory: copy before writing)."""
        e = self.entries[name]
        _, _, carrier = _DTYPES[_NAMES[e.dtype]]
        numel = int(np.prod(e.shape, dtype=np.int64)) if e.shape else 1
        if numel == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        arr = np.frombuffer(self._map, dtype=carrier, count=numel, offset=self.data_start + e.start)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)    # the mapping is read-only by design
            t = torch.from_numpy(arr)
        if e.dtype == torch.bfloat16:
            t = t.view(torch.bfloat16)
        return t.reshape(e.shape)

    def close(self) -> None:
        # Tensors handed out keep the map alive through numpy; dropping our references is enough.
        self._map = None
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    """Write CPU tensors in the order given."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of '{name}'")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + f".tmp{os.getpid()}"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, t in tensors.items():
            c = t.detach().contiguous().cpu()
            if c.dtype == torch.bfloat16:
                c = c.view(torch.int16)
            f.write(c.numpy().tobytes())
    os.replace(tmp, path)
