"""Reader of the safetensors container: 8-byte little-endian header length, that many bytes of
JSON {name: {dtype, shape, data_offsets}}, then the raw little-endian data.  Tensors are views of
one memory map, handed out one at a time so a checkpoint never sits in host memory twice."""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from typing import Dict, Iterator, Tuple

import torch

_DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
           "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
           "U8": torch.uint8, "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn,
           "F8_E5M2": torch.float8_e5m2}


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file")
        (n,) = struct.unpack("<Q", head)
        self.meta: Dict[str, dict] = json.loads(self._f.read(n).decode("utf-8"))
        self.meta.pop("__metadata__", None)
        self._base = 8 + n
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def keys(self):
        return list(self.meta)

    def shape(self, name: str):
        return tuple(self.meta[name]["shape"])

    def get(self, name: str) -> torch.Tensor:
        info = self.meta[name]
        if info["dtype"] not in _DTYPES:
            raise ValueError(f"{self.path}: tensor {name} has unsupported dtype {info['dtype']}")
        dt = _DTYPES[info["dtype"]]
        lo, hi = info["data_offsets"]
        count = 1
        for s in info["shape"]:
            count *= int(s)
        if (hi - lo) != count * torch.empty((), dtype=dt).element_size():
            raise ValueError(f"{self.path}: tensor {name}: size does not match its shape")
        if count == 0:
            return torch.empty(info["shape"], dtype=dt)
        buf = memoryview(self._map)[self._base + lo:self._base + hi]
        with warnings.catch_warnings():      # the map is read-only; the loader only copies out of it
            warnings.simplefilter("ignore", UserWarning)
            return torch.frombuffer(buf, dtype=dt, count=count).reshape(info["shape"])

    def items(self) -> Iterator[Tuple[str, torch.Tensor]]:
        for name in self.meta:
            yield name, self.get(name)

    def close(self):
        # tensors handed out keep views of the map alive; the map is released with them
        try:
            self._f.close()
        except OSError:
            pass
