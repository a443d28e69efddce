"""A small reader and writer of the safetensors container.

Layout of a file: an 8-byte little-endian header length ``n``, ``n`` bytes of
JSON ``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__"?}``,
then the raw little-endian tensor bytes; offsets count from the end of the
header.  This module plays the role the memory-mapped GGUF reader plays in the
reference (skyla-gguf/src/reader.rs:66-125): open, parse the header, check every
tensor against the end of the file, and hand out views by name.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One open file: ``names()``, ``info(name)`` and ``tensor(name)`` (a CPU view)."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: unexpected end of file (no header length)")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8:
            raise SafetensorsError(f"{path}: header of {n} bytes runs past end of file ({size} bytes)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not an object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + n
        self._data_len = size - self._data_start
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            try:
                dt, shape, (b, en) = e["dtype"], tuple(int(s) for s in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor {name!r}") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt}")
            numel = 1
            for s in shape:
                numel *= s
            if en - b != numel * _DTYPES[dt][1] or b < 0:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} of shape {list(shape)} {dt} does not fill its "
                    f"byte range [{b}, {en})")
            if en > self._data_len:
                raise SafetensorsError(f"{path}: tensor {name!r} runs past end of file")
            self._entries[name] = (dt, shape, b, en)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> Iterable[str]:
        return self._entries.keys()

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dt, shape, _, _ = self._entries[name]
        return _DTYPES[dt][0], shape

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only CPU tensor over the mapped bytes (copy before writing to it)."""
        dt, shape, b, en = self._entries[name]
        tdt = _DTYPES[dt][0]
        if en == b:
            return torch.empty(shape, dtype=tdt)
        buf = memoryview(self._mm)[self._data_start + b:self._data_start + en]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the buffer is read-only; callers copy
            t = torch.frombuffer(buf, dtype=tdt)
        return t.view(shape)

    def close(self):
        # views may still reference the map; leave unmapping to the garbage collector
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Write CPU tensors in name order, each aligned to 8 bytes through header padding."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    blobs = []
    for name in order:
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} ({name})")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        blobs.append(t)
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for t in blobs:
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())
