"""Reading and writing the safetensors container, without any library for it.

File layout: an unsigned 64-bit little-endian header length, a JSON header
``name -> {dtype, shape, data_offsets}`` (offsets relative to the end of the
header), then the raw little-endian tensor bytes.  The reference's container is
GGUF (src/gguf.c:176-266); its discipline is kept: every length and offset is
checked against the file before any byte is touched (src/gguf.c:614-650).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
MAX_HEADER_BYTES = 100 * 1024 * 1024


class SafetensorsError(ValueError):
    pass


class TensorEntry:
    __slots__ = ("name", "dtype", "shape", "begin", "end")

    def __init__(self, name: str, dtype: str, shape: Tuple[int, ...], begin: int, end: int):
        self.name, self.dtype, self.shape, self.begin, self.end = name, dtype, shape, begin, end


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are read one at a time by name."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"'{path}' is too short to be a safetensors file ({size} bytes)")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > MAX_HEADER_BYTES or 8 + hlen > size:
            raise SafetensorsError(f"'{path}': header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"'{path}': header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"'{path}': header must be a JSON object")
        self.data_start = 8 + hlen
        data_len = size - self.data_start
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                dtype, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"'{path}': malformed entry for tensor '{name}'") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"'{path}': tensor '{name}' has unsupported dtype {dtype}")
            n = 1
            for s in shape:
                if s < 0:
                    raise SafetensorsError(f"'{path}': tensor '{name}' has a negative dimension")
                n *= s
            if not (0 <= b <= e <= data_len) or e - b != n * _DTYPES[dtype][1]:
                raise SafetensorsError(
                    f"'{path}': tensor '{name}' claims bytes [{b}, {e}) for shape {list(shape)} "
                    f"{dtype}; the data section holds {data_len} bytes")
            self.entries[name] = TensorEntry(name, dtype, shape, b, e)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> List[str]:
        return list(self.entries)

    def read(self, name: str) -> torch.Tensor:
        """The tensor as a CPU tensor that owns its memory."""
        e = self.entries[name]
        dtype, _ = _DTYPES[e.dtype]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=dtype)
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=e.end - e.begin, offset=self.data_start + e.begin)
        return torch.from_numpy(buf.copy()).view(dtype).reshape(e.shape)

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def _raw_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous()
    return t.view(torch.uint8).numpy().tobytes() if t.numel() else b""


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata: Dict[str, str] = None) -> None:
    """Write ``(name, tensor)`` pairs.  The pairs are consumed twice when given as a
    list; a generator is materialised tensor by tensor into a temporary data file first."""
    tmp_data = path + ".data.tmp"
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    with open(tmp_data, "wb") as df:
        for name, t in tensors:
            if name in header:
                raise SafetensorsError(f"tensor '{name}' is written twice")
            if t.dtype not in _NAMES:
                raise SafetensorsError(f"tensor '{name}' has unsupported dtype {t.dtype}")
            raw = _raw_bytes(t)
            header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                            "data_offsets": [offset, offset + len(raw)]}
            df.write(raw)
            offset += len(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    with open(path, "wb") as out, open(tmp_data, "rb") as df:
        out.write(struct.pack("<Q", len(hjson)))
        out.write(hjson)
        while True:
            chunk = df.read(1 << 24)
            if not chunk:
                break
            out.write(chunk)
    os.remove(tmp_data)
