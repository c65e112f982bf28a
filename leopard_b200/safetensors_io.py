"""Reader / writer of the safetensors container: 8-byte little-endian header length, a JSON header {name: {dtype, shape,
data_offsets}}, then the raw little-endian data.  Only what the checkpoint loaders of this package need: BF16, F32, F16, I32, I64.
The file is memory-mapped; tensors are materialised one at a time, so a loader can stream a checkpoint to the device layer by layer."""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterable, Tuple

import torch

_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "I64": torch.int64}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    def __init__(self, path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise ValueError(f"{self.path}: not a safetensors file")
        (n,) = struct.unpack("<Q", head)
        self.meta = json.loads(self._f.read(n))
        self.meta.pop("__metadata__", None)
        self._base = 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def keys(self) -> Iterable[str]:
        return self.meta.keys()

    def __contains__(self, name: str) -> bool:
        return name in self.meta

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.meta[name]["shape"])

    def __getitem__(self, name: str) -> torch.Tensor:
        try:
            m = self.meta[name]
        except KeyError:
            raise KeyError(f"{self.path}: no tensor named {name!r}") from None
        dt = _DTYPES.get(m["dtype"])
        if dt is None:
            raise ValueError(f"{self.path}: tensor {name!r} has unsupported dtype {m['dtype']}")
        a, b = m["data_offsets"]
        raw = bytearray(self._mm[self._base + a:self._base + b])   # a private copy: the tensor outlives the mapping
        if not raw:
            return torch.empty(m["shape"], dtype=dt)
        return torch.frombuffer(raw, dtype=dt).reshape(m["shape"])

    def close(self):
        self._mm.close()
        self._f.close()


def save_file(tensors: Dict[str, torch.Tensor], path) -> None:
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    head = json.dumps(header, separators=(",", ":")).encode()
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for raw in blobs:
            f.write(raw)
