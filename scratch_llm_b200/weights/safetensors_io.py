"""Reading and writing ``.safetensors`` files: an 8-byte little-endian header length, a JSON
header ``{name: {dtype, shape, data_offsets}}``, then the raw little-endian tensor bytes.

The reference stores weights as a ``torch.save`` pickle (src/scratch_llm/train.py:101-127) and
states that it has no safetensors loader (src/scratch_llm/serving/loadgen.py:35-36); this file
is the engine's own reader, keyed by tensor name.
"""

from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Iterator, Mapping

import torch

_DTYPES: dict[str, torch.dtype] = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    """A memory-mapped safetensors file.  ``entries`` lists what it holds without reading any
    tensor; :meth:`tensor` returns a CPU tensor that views the mapping."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: too short to be a safetensors file")
        self._file = open(self.path, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_COPY)
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if 8 + header_len > size:
            raise SafetensorsError(f"{self.path}: header length {header_len} runs past the "
                                   f"end of the file ({size} bytes)")
        try:
            header = json.loads(self._map[8:8 + header_len].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{self.path}: header is not JSON: {exc}") from None
        self._data_start = 8 + header_len
        self.metadata: Mapping[str, str] = header.pop("__metadata__", {}) or {}
        self.entries: dict[str, TensorEntry] = {}
        for name, info in header.items():
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has unsupported dtype "
                                       f"{info['dtype']!r}")
            dtype = _DTYPES[info["dtype"]]
            shape = tuple(int(s) for s in info["shape"])
            begin, end = (int(x) for x in info["data_offsets"])
            numel = 1
            for s in shape:
                numel *= s
            if end - begin != numel * dtype.itemsize:
                raise SafetensorsError(f"{self.path}: tensor {name!r} of shape {shape} and "
                                       f"dtype {info['dtype']} spans {end - begin} bytes")
            if begin < 0 or self._data_start + end > size:
                raise SafetensorsError(f"{self.path}: tensor {name!r} ends at byte "
                                       f"{self._data_start + end}, past the end of the file "
                                       f"({size} bytes): the file is truncated")
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end)

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        numel = (e.end - e.begin) // e.dtype.itemsize
        if numel == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        flat = torch.frombuffer(self._map, dtype=e.dtype, count=numel,
                                offset=self._data_start + e.begin)
        return flat.view(e.shape)

    def __iter__(self) -> Iterator[str]:
        return iter(self.entries)

    def close(self) -> None:
        # tensors handed out view the mapping; closing is left to the garbage collector when
        # any are alive
        try:
            self._map.close()
        except BufferError:
            pass
        self._file.close()


def write_safetensors(path: str | Path, tensors: Mapping[str, torch.Tensor],
                      metadata: Mapping[str, str] | None = None) -> Path:
    """Write ``tensors`` (any device) in name order, each tensor's bytes 8-byte aligned by a
    padded header."""
    path = Path(path)
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    names = sorted(tensors)
    for name in names:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r} has dtype {t.dtype}, which safetensors "
                                   "cannot store")
        nbytes = t.numel() * t.dtype.itemsize
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((-(8 + len(blob))) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in names:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())
    return path
