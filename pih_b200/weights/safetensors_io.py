"""Reader and writer of the safetensors container, by tensor name.

Format rules as the reference's parser enforces them
(src/model/safetensors_header.cpp:90-159; record checks :34-86; dtypes
:12-24): an 8-byte little-endian header length, a JSON header mapping each
name to ``{dtype, shape, data_offsets}``, then the payload; a tensor's byte
count equals the product of its shape times the element size, and the
ranges tile the payload without gap or overlap.  Files are memory-mapped;
``read_tensor`` returns a torch tensor that owns a copy.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4), "I64": (torch.int64, 8), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1), "F64": (torch.float64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 16 * 1024 * 1024


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorRecord:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: shorter than the 8-byte header length")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} is out of bounds")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self._data_start = 8 + hlen
        payload = size - self._data_start
        self.records: Dict[str, TensorRecord] = {}
        for name, rec in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype, esize = _DTYPES[rec["dtype"]]
                shape = tuple(int(x) for x in rec["shape"])
                begin, end = (int(x) for x in rec["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: bad record for tensor {name!r}: {rec!r}") from None
            count = 1
            for s in shape:
                if s < 0:
                    raise SafetensorsError(f"{path}: tensor {name!r} has a negative extent")
                count *= s
            if end - begin != count * esize or begin < 0 or end > payload:
                raise SafetensorsError(f"{path}: tensor {name!r}: {end - begin} bytes do not match "
                                       f"shape {shape} of {rec['dtype']}")
            self.records[name] = TensorRecord(name, dtype, shape, begin, end)
        cursor = 0
        for rec in sorted(self.records.values(), key=lambda r: (r.begin, r.end)):
            if rec.begin != cursor:
                raise SafetensorsError(f"{path}: payload has a gap or overlap before tensor {rec.name!r}")
            cursor = rec.end
        if cursor != payload:
            raise SafetensorsError(f"{path}: {payload - cursor} payload bytes belong to no tensor")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> Iterable[str]:
        return self.records.keys()

    def read_tensor(self, name: str) -> torch.Tensor:
        rec = self.records[name]
        view = memoryview(self._mm)[self._data_start + rec.begin:self._data_start + rec.end]
        if rec.end == rec.begin:
            return torch.empty(rec.shape, dtype=rec.dtype)
        flat = torch.frombuffer(bytearray(view), dtype=torch.uint8)
        return flat.view(rec.dtype).reshape(rec.shape)

    def close(self) -> None:
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass
            self._mm = None
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """Write ``tensors`` in sorted-name order (payload tiled without gaps)."""
    header = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
