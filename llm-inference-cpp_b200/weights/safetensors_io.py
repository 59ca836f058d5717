"""Reading and writing one ``model.safetensors`` file.

File format as the reference parses it (src/model/safetensors.cpp:116-223): an
8-byte little-endian header length, a JSON header mapping each tensor name to
``{"dtype", "shape", "data_offsets"}`` (plus an optional ``__metadata__``), then
the tensor bytes.  The same refusals are kept: short file, oversize header,
header past the end, unknown dtype or field, offsets that do not match
dtype × shape, overlapping tensors, holes and trailing bytes.

Tensors are returned as views of a read-only memory map; nothing is converted
here.  Storage types map to torch as: F32→float32, BF16→bfloat16, F16→float16,
I32→int32, I64→int64 (the loader narrows integer tables to int32), and the small
integer/bool types for completeness of error messages.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass

import numpy as np
import torch

MAX_HEADER_BYTES = 100 * 1000 * 1000
MAX_TENSORS = 1 << 20
MAX_RANK = 8
MAX_NAME = 1024

_DTYPES = {
    "F64": (8, torch.float64, np.float64), "F32": (4, torch.float32, np.float32),
    "F16": (2, torch.float16, np.float16), "BF16": (2, torch.bfloat16, np.uint16),
    "I64": (8, torch.int64, np.int64), "I32": (4, torch.int32, np.int32),
    "I16": (2, torch.int16, np.int16), "I8": (1, torch.int8, np.int8),
    "U8": (1, torch.uint8, np.uint8), "BOOL": (1, torch.bool, np.bool_),
}
_TORCH_TO_NAME = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.int32: "I32",
                  torch.int64: "I64", torch.float64: "F64"}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: tuple
    begin: int
    end: int

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class SafetensorsFile:
    """A parsed safetensors file; ``tensor(name)`` gives a torch view of the mapped bytes."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            self._f = open(path, "rb")
        except OSError:
            raise SafetensorsError(f"cannot open {path}") from None
        if size < 8:
            raise SafetensorsError(f"{path}: file too short for a safetensors header")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > MAX_HEADER_BYTES:
            raise SafetensorsError(f"{path}: header of {hlen} bytes is larger than {MAX_HEADER_BYTES}")
        if 8 + hlen > size:
            raise SafetensorsError(f"{path}: header runs past the end of the file")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"), object_pairs_hook=self._no_dups)
        except (ValueError, UnicodeDecodeError) as e:
            raise SafetensorsError(f"{path}: bad header: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not a JSON object")
        self.data_start = 8 + hlen
        self.data_len = size - self.data_start
        self.metadata = header.pop("__metadata__", None)
        if len(header) > MAX_TENSORS:
            raise SafetensorsError(f"{path}: too many tensors")
        infos = [self._parse_entry(n, e) for n, e in header.items()]
        infos.sort(key=lambda t: t.begin)
        cursor = 0
        for t in infos:
            if t.begin < cursor:
                raise SafetensorsError(f"{path}: tensor {t.name} overlaps another tensor")
            if t.begin > cursor:
                raise SafetensorsError(f"{path}: hole in the data before tensor {t.name}")
            cursor = t.end
        if cursor != self.data_len:
            raise SafetensorsError(f"{path}: {self.data_len - cursor} trailing bytes after the last tensor")
        self.tensors = {t.name: t for t in sorted(infos, key=lambda t: t.name)}
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    @staticmethod
    def _no_dups(pairs):
        d = {}
        for k, v in pairs:
            if k in d:
                raise ValueError(f'duplicate key "{k}"')
            d[k] = v
        return d

    def _parse_entry(self, name, e) -> TensorInfo:
        p = self.path
        if len(name) > MAX_NAME:
            raise SafetensorsError(f"{p}: tensor name longer than {MAX_NAME}")
        if not isinstance(e, dict) or set(e) != {"dtype", "shape", "data_offsets"}:
            raise SafetensorsError(f"{p}: tensor {name} must have exactly dtype, shape and data_offsets")
        if e["dtype"] not in _DTYPES:
            raise SafetensorsError(f"{p}: tensor {name} has unknown dtype {e['dtype']}")
        shape = e["shape"]
        if (not isinstance(shape, list) or len(shape) > MAX_RANK
                or any(isinstance(s, bool) or not isinstance(s, int) or s < 0 for s in shape)):
            raise SafetensorsError(f"{p}: tensor {name} has a bad shape")
        off = e["data_offsets"]
        if (not isinstance(off, list) or len(off) != 2
                or any(isinstance(o, bool) or not isinstance(o, int) or o < 0 for o in off)
                or off[0] > off[1] or off[1] > self.data_len):
            raise SafetensorsError(f"{p}: tensor {name} has bad data_offsets")
        n = 1
        for s in shape:
            n *= s
        if n * _DTYPES[e["dtype"]][0] != off[1] - off[0]:
            raise SafetensorsError(f"{p}: tensor {name}: {off[1] - off[0]} bytes do not match dtype × shape")
        return TensorInfo(name, e["dtype"], tuple(shape), off[0], off[1])

    def names(self) -> list[str]:
        return list(self.tensors)

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only CPU tensor viewing the file's bytes (storage dtype kept)."""
        t = self.tensors[name]
        _, tdt, ndt = _DTYPES[t.dtype]
        if t.numel == 0:
            return torch.empty(t.shape, dtype=tdt)
        arr = np.frombuffer(self._map, dtype=ndt, count=t.numel, offset=self.data_start + t.begin)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; nobody writes through the view
            out = torch.from_numpy(arr)
        if t.dtype == "BF16":
            out = out.view(torch.bfloat16)
        return out.reshape(t.shape)

    def parameter_count(self) -> int:
        return sum(t.numel for t in self.tensors.values())

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        self._f.close()


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """Write CPU torch tensors (name → tensor) as one safetensors file, names sorted."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TORCH_TO_NAME:
            raise SafetensorsError(f"cannot write dtype {t.dtype} of tensor {name}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            f.write(t.numpy().tobytes())
